"""Batatar on the host: config.json through the registry's parser (every key, defaults, refusals, the run order of a looped
block) and the plain restatement against itself (a whole prompt equals portions and token-by-token decoding).  No GPU."""
import ctypes as C
import importlib
import json

import pytest
import torch

from oracle import batatar_oracle as B


@pytest.fixture(scope="module")
def lib():
    return importlib.import_module("nano-vllm-candle_b200._lib").lib()


def parse(lib, cfg):
    h = C.c_void_p()
    rc = lib.nvc_model_config_from_json(json.dumps(cfg).encode(), C.byref(h))
    return rc, h, lib.nvc_model_config_last_error().decode()


def good(loop=(1, 3, 2)):
    return B.make_config(vocab=77, width=40, residual_mult=0.4, loop=loop, layers=[
        B.with_moe(B.parallel_cfg(), 5, 2, 24),
        B.with_moe(B.lightning_cfg(), 3, 1, 16),
        B.with_moe(B.parallel_cfg(heads=2, kv_heads=2, dim=8, vdim=12, chunk=5, s_heads=2, s_groups=1, conv=2, norm_groups=1), None),
        B.with_moe(B.lightning_cfg(heads=2), 4, 4, 8),
    ])


def runs(lib, h, n=16):
    layers, passes, opens = (C.c_int32 * n)(), (C.c_int32 * n)(), (C.c_int32 * n)()
    k = lib.nvc_model_config_layer_runs(h, layers, passes, opens, n)
    return list(zip(list(layers)[:k], list(passes)[:k], list(opens)[:k]))


def test_a_configuration_is_accepted_and_registered(lib):
    rc, h, err = parse(lib, good())
    assert rc == 0, err
    assert lib.nvc_model_config_architecture(h).decode() == "Batatar"
    assert lib.nvc_model_config_vocab(h) == 77
    assert runs(lib, h) == [(0, 0, 0), (1, 0, 1), (2, 0, 0), (1, 1, 1), (2, 1, 0), (3, 0, 0)]
    assert runs(lib, h) == [(i, t, int(o)) for i, t, o in B.layer_runs(good())]
    lib.nvc_model_config_free(h)


@pytest.mark.parametrize("loop", [None, (0, 4, 1), (0, 1, 3), (3, 4, 2)])
def test_run_order_of_other_loops(lib, loop):
    rc, h, err = parse(lib, good(loop))
    assert rc == 0, err
    assert runs(lib, h) == [(i, t, int(o)) for i, t, o in B.layer_runs(good(loop))]
    lib.nvc_model_config_free(h)


def broken(mutate):
    c = good()
    mutate(c)
    return c


@pytest.mark.parametrize("mutate,needle", [
    (lambda c: c["layers"][0].update(type="attention"), "not supported"),
    (lambda c: c["layers"][0]["mixer"].pop("left"), "left"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(softcap=-1.0), "softcap"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=0), "mask"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("state"), "state"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(groups=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(conv=40), "taps"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5, 1.5, 0.2]), "decay"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=8), "top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="dense"), "not supported"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(start=3, stop=3), "loop"),
    (lambda c: c["loop"].update(times=0), "times"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c.pop("norm"), "norm.eps"),
])
def test_what_the_parser_refuses(lib, mutate, needle):
    rc, h, err = parse(lib, broken(mutate))
    assert rc != 0 and needle in err, err


def test_absent_keys_mean_absent_mechanisms(lib):
    c = good()
    c["layers"][0]["mixer"]["left"].pop("softcap")          # scores are not capped
    c["layers"][0]["mixer"]["left"].pop("mask")             # every earlier token is visible
    c["layers"][3]["mlp"] = None
    c.pop("loop")                                            # every layer runs once, no pass opens
    rc, h, err = parse(lib, c)
    assert rc == 0, err
    assert runs(lib, h) == [(i, 0, 0) for i in range(4)]
    lib.nvc_model_config_free(h)


def test_the_restatement_agrees_with_itself_however_the_prompt_is_cut():
    cfg = good()
    m = B.Batatar(cfg, B.make_weights(cfg, 3))
    p = torch.randint(0, 77, (40,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = m.forward(p)
    for sizes in ([1] * 40, [2, 3, 1, 11, 5, 18], [39, 1]):
        cache, rows, at = m.new_cache(), [], 0
        for n in sizes:
            rows.append(m.forward(p[at:at + n], cache))
            at += n
        assert (torch.cat(rows) - whole).abs().max() < 2e-4
