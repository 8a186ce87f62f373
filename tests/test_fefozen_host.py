"""Fefozen on the host: config.json through the registry's parser (every key, defaults, refusals).  No GPU."""
import ctypes as C
import importlib
import json

import pytest

from oracle import fefozen_oracle as F


@pytest.fixture(scope="module")
def lib():
    return importlib.import_module("nano-vllm-candle_b200._lib").lib()


def parse(lib, cfg):
    h = C.c_void_p()
    rc = lib.nvc_model_config_from_json(json.dumps(cfg).encode(), C.byref(h))
    return rc, h, lib.nvc_model_config_last_error().decode()


def good():
    return F.make_config(vocab=77, width=40, layers=[
        F.with_dense(F.latent_cfg(second=True), 64),
        F.with_moe(F.latent_cfg(), 5, 2, 2, 24),
        F.with_dense(F.latent_cfg(second=True, kv_from=0, heads=2, dim=8, vdim=12), None),
        F.with_moe(F.delta_cfg(), 3, 0, 1, 16),
    ])


def test_a_configuration_is_accepted_and_registered(lib):
    rc, h, err = parse(lib, good())
    assert rc == 0, err
    assert lib.nvc_model_config_architecture(h).decode() == "Fefozen"
    assert lib.nvc_model_config_vocab(h) == 77
    layers = (C.c_int32 * 8)()
    assert lib.nvc_model_config_layer_runs(h, layers, None, None, 8) == 4 and list(layers)[:4] == [0, 1, 2, 3]
    lib.nvc_model_config_free(h)


def broken(mutate):
    c = good()
    mutate(c)
    return c


@pytest.mark.parametrize("mutate,needle", [
    (lambda c: c["layers"][0].update(type="attention"), "not supported"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"].pop("rot_dim"), "rot_dim"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rot.dims"),                 # more rotated numbers than the part has
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "earlier"),                       # itself
    (lambda c: c["layers"][2]["mixer"].update(kv_from=3), "earlier"),                       # a later layer
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "must equal"),                    # another kind of rotation and other sizes
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=24), "must equal"),
    (lambda c: c["layers"].append(F.with_dense(F.latent_cfg(second=True, kv_from=2, heads=2, dim=8, vdim=12), None)), "cache of its own"),
    (lambda c: c["layers"][3]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][3]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=8), "top"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "not supported"),
    (lambda c: c.pop("norm"), "norm.eps"),
])
def test_what_the_parser_refuses(lib, mutate, needle):
    rc, h, err = parse(lib, broken(mutate))
    assert rc != 0 and needle in err, err


def test_absent_keys_mean_absent_mechanisms(lib):
    c = good()
    c["layers"][3]["mlp"]["router"].pop("identity")          # no identity experts
    c["layers"][0]["mixer"]["rot_dim"] = 0                    # no rotated part: no `rot` needed
    c["layers"][0]["mixer"].pop("rot")
    c["layers"][2]["mixer"].pop("kv_from")                    # its own rows again (sizes no longer tied to layer 0)
    c["layers"][0]["mlp"] = None
    rc, h, err = parse(lib, c)
    assert rc == 0, err
    lib.nvc_model_config_free(h)
