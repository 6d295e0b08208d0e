"""Porarax without a GPU: the configuration's checks, what the builder makes of a configuration (parts, tensor names and
shapes, run order, how far back a shared latent is kept), padded heads of a stacked projection, and the plain
implementation's mechanisms against restatements of their own definitions."""
import copy

import numpy as np
import pytest
import torch

from tinyllama_c_b200.config import ConfigError, config_from_dict
from tinyllama_c_b200.config.base import lookup_architecture
from tinyllama_c_b200.parts.base import KVRequest, StateRequest
from tinyllama_c_b200.parts.linear import StackedLinear

import configs
from plain import porarax_plain as plain


def build(cfg: dict):
    c = config_from_dict(cfg)
    return lookup_architecture(c.architecture)[1](c)


def test_builder_names_shapes_and_run_order():
    m = build(configs.PORARAX_A)
    got = {s.name: tuple(s.shape) for s in m.weight_specs()}
    assert got["embed"] == (150, 64) and got["final.norm"] == (64,) and got["l0.norm1"] == (64,)
    # delta: 2 query/key heads of 16, 4 value heads of 24, 3 taps
    assert got["l0.mix.q"] == (32, 64) and got["l0.mix.q.conv"] == (32, 3) and got["l0.mix.v"] == (96, 64)
    assert got["l0.mix.v.conv"] == (96, 3) and got["l0.mix.b"] == (4, 64) and got["l0.mix.A_log"] == (4,)
    assert got["l0.mix.norm"] == (24,) and got["l0.mix.g"] == (96, 64) and got["l0.mix.o"] == (64, 96)
    # latent attention: the query's latent, the shared latent, per-head up-projections
    assert got["l1.mix.dq"] == (24, 64) and got["l1.mix.dq.norm"] == (24,) and got["l1.mix.uq"] == (48, 24)
    assert got["l1.mix.dkv"] == (32, 64) and got["l1.mix.uk"] == (48, 32) and got["l1.mix.uv"] == (24, 32)
    assert "l3.mix.dkv" not in got and "l3.mix.dkv.norm" not in got and got["l3.mix.uk"] == (16, 32)
    # attention with values wider than keys: the stored shapes are the unpadded ones
    assert got["l4.mix.q"] == (96, 64) and got["l4.mix.k"] == (16, 64) and got["l4.mix.v"] == (40, 64)
    assert got["l4.mix.g"] == (240, 64) and got["l4.mix.o"] == (64, 240)
    assert got["l4.mlp.router"] == (6, 64) and got["l4.mlp.router.b"] == (6,) and got["l4.mlp.e5.down"] == (64, 8)
    assert not any(n.startswith("l2.mlp") for n in got)
    assert [(r.layer, r.kv_cache) for r in m.schedule] == [(0, None), (1, None), (2, None), (3, 1), (4, None)]
    reqs = m.cache_requests()
    assert reqs[3] == [] and reqs[1] == [KVRequest("latent", 1, 32, 100, values=False)]        # the reader's wider window
    assert StateRequest("delta.state", (4, 16, 24)) in reqs[0] and StateRequest("delta.conv", (2, 2 * 32 + 96)) in reqs[0]
    assert reqs[4] == [KVRequest("kv", 1, 40, None)]
    # a feed-forward without a norm of its own is the parallel branch
    assert all(b.parallel_ffn == (b.ffn is not None) for b in m.layers) and m.layers[2].ffn is None
    b = build(configs.PORARAX_B)
    assert b.cache_requests()[3] == [KVRequest("latent", 1, 20, 64, values=False)]             # the owner's window is wider


@pytest.mark.parametrize("edit,text", [
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=16), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"].pop("mask"), "mask"),
    (lambda c: c["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=7), "rot"),
    (lambda c: c["layers"][2]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "router"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configuration_faults_are_named(edit, text):
    cfg = copy.deepcopy(configs.PORARAX_A)
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(cfg)


def test_padded_heads_of_a_stacked_projection():
    g = torch.Generator().manual_seed(1)
    D, n, have, want = 10, 3, 4, 6
    w = torch.randn(n * have, D, generator=g)
    lin = StackedLinear(D)
    lin.add("w", n * want, heads=(n, have, want))
    assert lin.weight_specs()[0].shape == (n * have, D)
    laid = lin._laid_out(lin.segments[0], w).reshape(n, want, D)
    assert torch.equal(laid[:, :have], w.reshape(n, have, D)) and not laid[:, have:].any()
    out = StackedLinear(n * want, in_heads=(n, have, want))
    out.add("o", 7)
    wo = torch.randn(7, n * have, generator=g)
    assert out.weight_specs()[0].shape == (7, n * have)
    laid = out._laid_out(out.segments[0], wo).reshape(7, n, want)
    assert torch.equal(laid[:, :, :have], wo.reshape(7, n, have)) and not laid[:, :, have:].any()
    x = torch.randn(5, n, have, generator=g)
    padded = torch.zeros(5, n, want)
    padded[:, :, :have] = x
    assert torch.allclose(padded.reshape(5, -1) @ out._laid_out(out.segments[0], wo).T, x.reshape(5, -1) @ wo.T, atol=1e-6)


def test_plain_delta_rule_is_the_least_squares_step_it_claims_to_be():
    """With decay 1 and beta 1 a write makes the state return exactly the written value for its key; an orthogonal key's
    value is left alone."""
    g = np.random.default_rng(2)
    dk, dv = 6, 4
    k1 = np.zeros(dk); k1[0] = 1.0
    k2 = np.zeros(dk); k2[3] = 1.0
    v1, v2, v3 = g.standard_normal(dv), g.standard_normal(dv), g.standard_normal(dv)
    S = np.zeros((dk, dv))
    for k, v in ((k1, v1), (k2, v2), (k1, v3)):
        S = S + np.outer(k, 1.0 * (v - S.T @ k))
    assert np.allclose(S.T @ k1, v3) and np.allclose(S.T @ k2, v2)


def test_plain_window_and_routing():
    g = np.random.default_rng(3)
    order, w = plain.route(np.array([0.5, 2.0, 2.0, -1.0]), 3)
    assert order == [1, 2, 0] and np.isclose(w.sum(), 1.0) and np.isclose(w[0], w[1])
    # a window of one key: every row attends to itself alone, so the mixer is a per-token map
    D, H, dn, dv, R, qr = 8, 2, 4, 3, 5, 6
    W = {"a.dq": g.standard_normal((qr, D)), "a.dq.norm": np.ones(qr), "a.uq": g.standard_normal((H * dn, qr)),
         "a.dkv": g.standard_normal((R, D)), "a.dkv.norm": np.ones(R), "a.uk": g.standard_normal((H * dn, R)),
         "a.uv": g.standard_normal((H * dv, R)), "a.o": g.standard_normal((D, H * dv))}
    m = dict(heads=H, dim=dn, vdim=dv, kv_rank=R, q_rank=qr, scale=0.3, mask=dict(size=1))
    h = g.standard_normal((7, D))
    c = plain.latent_rows(h, W, "a.", 1e-5)
    full = plain.latent_attention(h, W, "a.", m, c, 1e-5)
    assert np.allclose(full, (c @ W["a.uv"].T) @ W["a.o"].T)
    # a window as long as the sequence equals no window; one shorter changes the last row only
    m7, m6 = dict(m, mask=dict(size=7)), dict(m, mask=dict(size=6))
    a, b = plain.latent_attention(h, W, "a.", m7, c, 1e-5), plain.latent_attention(h, W, "a.", m6, c, 1e-5)
    assert np.allclose(a[:6], b[:6]) and not np.allclose(a[6], b[6])
