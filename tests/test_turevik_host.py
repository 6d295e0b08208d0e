"""Turevik without a GPU: configuration (both spellings of the architecture key, what is refused), the model's declared
tensors and run order, a cache whose key pages have no values and whose entries read another entry's keys, the plain
implementation's pieces against each other."""
import copy

import numpy as np
import pytest
import torch

import tinyllama_c_b200 as tlc
from tinyllama_c_b200.cache import Cache
from tinyllama_c_b200.config import ConfigError, config_from_dict
from tinyllama_c_b200.parts.base import KVRequest, LayerRun, StateRequest
from tinyllama_c_b200.weights.loader import build_model

import configs
from plain import turevik_plain as plain


def test_configuration_reads_every_layer_and_says_what_is_wrong():
    cfg = config_from_dict(copy.deepcopy(configs.TUREVIK_A))
    assert cfg.architecture == "Turevik" and cfg.width == 64 and len(cfg.layers) == 5 and cfg.eps == 1e-5
    assert config_from_dict(cfg.to_dict()) == cfg
    for change, word in [(lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 0), "kv_from"),      # layer 0 is recurrent
                         (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 3), "kv_from"),      # a later layer
                         (lambda c: c["layers"][2]["mixer"].__setitem__("kv_rank", 16), "kv_rank"),
                         (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 18), "rot"),
                         (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top"),
                         (lambda c: c["layers"][4].__setitem__("type", "conv"), "type"),
                         (lambda c: c.__setitem__("norm", {}), "eps")]:
        bad = copy.deepcopy(configs.TUREVIK_A)
        change(bad)
        with pytest.raises(ConfigError, match=word):
            config_from_dict(bad)
    with pytest.raises(ConfigError):
        config_from_dict({"architecture": "NoSuchDesign"})


def test_declared_tensors_run_order_and_cache_needs():
    model = build_model(config_from_dict(copy.deepcopy(configs.TUREVIK_A)))
    names = {s.name: tuple(s.shape) for s in model.weight_specs()}
    assert names["embed"] == (160, 64) and names["final.norm"] == (64,) and names["l0.shift"] == (64,)
    assert names["l1.mix.dkv"] == (32 + 16, 64) and names["l1.mix.q"] == (3 * (8 + 16), 64) and names["l1.mix.sink"] == (3,)
    assert "l2.mix.dkv" not in names and "l2.mix.dkv.norm" not in names and names["l2.mix.uk"] == (2 * 16, 32)
    assert names["l0.mlp.e5.down"] == (64, 24) and names["l0.mlp.shared.sg"] == (1, 64) and names["l0.mix.z.b"] == (48,)
    assert not any(n.startswith("l2.mlp") for n in names) and "l3.mlp.shared.gate" not in names
    assert model.schedule == [LayerRun(0), LayerRun(1), LayerRun(2, kv_cache=1), LayerRun(3), LayerRun(4)]
    needs = model.cache_requests()
    assert [type(q) for q in needs[2]] == [StateRequest]                       # its keys are entry 1's
    assert any(isinstance(q, KVRequest) and not q.values and q.head_dim == 48 for q in needs[1])
    assert {q.key for q in needs[0]} == {"shift", "mingru"}


def test_cache_without_values_and_an_entry_that_reads_anothers_keys():
    reqs = {0: [KVRequest("latent", 1, 24, None, values=False), StateRequest("shift", (8,))],
            1: [StateRequest("shift", (8,))], 2: [KVRequest("kv", 2, 12)]}
    c = Cache(reqs, max_tokens=256, max_seqs=3, dtype=torch.float32, device="cpu")
    assert len(c.kv_groups) == 2 and c.kv_groups[0].v is None and c.kv_groups[1].v is not None
    own, reader = c.layer_view(0), c.layer_view(1, True, 0)
    assert reader.kv["latent"].k_pages.data_ptr() == own.kv["latent"].k_pages.data_ptr() and reader.kv["latent"].v_pages is None
    assert reader.state["shift"].data_ptr() != own.state["shift"].data_ptr()
    assert own.kv_writes and reader.writes and not reader.kv_writes
    s = c.acquire()
    c.reserve(s, 70)
    c.commit(s, 70)
    assert c.kv_groups[0].pool.n_held == 2 and c.kv_groups[1].pool.n_held == 2
    c.release(s)
    c.check()


def test_run_order_refuses_keys_of_a_later_or_borrowing_entry():
    from tinyllama_c_b200.models.model import Model
    cfg = config_from_dict(copy.deepcopy(configs.TUREVIK_A))
    model = build_model(cfg)
    specs = [b.spec for b in model.layers]
    norm = tlc.PartSpec("norm", "rmsnorm", dict(width=64, eps=1e-5, weight_name="final.norm", offset=1.0))
    for order in ([LayerRun(0), LayerRun(1, kv_cache=3), LayerRun(2), LayerRun(3), LayerRun(4)],
                  [LayerRun(0), LayerRun(1), LayerRun(2, kv_cache=1), LayerRun(3, kv_cache=2), LayerRun(4)]):
        with pytest.raises(ValueError, match="keys and values"):
            Model(cfg, specs, order, norm, "embed", None, 160, 64)


def test_plain_pieces_agree_with_each_other():
    """The recurrence carried over a cut equals the whole; the shift with a kept row equals the whole; attention in the
    latent space equals attention over built keys and values."""
    g = np.random.default_rng(0)
    D, Wd = 12, 20
    W = {"m.z": g.standard_normal((Wd, D)), "m.x": g.standard_normal((Wd, D)), "m.g": g.standard_normal((Wd, D)),
         "m.o": g.standard_normal((D, Wd)), "m.z.b": g.standard_normal(Wd), "m.x.b": g.standard_normal(Wd)}
    h = g.standard_normal((9, D))
    whole, _ = plain.mingru(h, W, "m.")
    a, S = plain.mingru(h[:4], W, "m.")
    b, _ = plain.mingru(h[4:], W, "m.", state=S)
    assert np.allclose(np.concatenate([a, b]), whole)
    mu = g.random(D)
    assert np.allclose(np.concatenate([plain.token_shift(h[:4], mu), plain.token_shift(h[4:], mu, before=h[3])]), plain.token_shift(h, mu))
    H, dn, r, dv, R = 2, 6, 4, 5, 8
    m = dict(heads=H, dim=dn, rot_dim=r, vdim=dv, kv_rank=R, scale=0.4, rot=dict(base=100.0, dims=4))
    W = {"a.q": g.standard_normal((H * (dn + r), D)), "a.dkv": g.standard_normal((R + r, D)), "a.dkv.norm": g.random(R) + 0.5,
         "a.uk": g.standard_normal((H * dn, R)), "a.uv": g.standard_normal((H * dv, R)), "a.sink": g.standard_normal(H),
         "a.o": np.eye(H * dv)}
    pos = np.arange(9)
    c, kr = plain.latent_cache_rows(h, W, "a.", m, 1e-6, pos)
    want = plain.latent_attention(h, W, "a.", m, pos, c, kr).reshape(9, H, dv)
    q = (h @ W["a.q"].T).reshape(9, H, dn + r)
    qr = plain.rotate_interleaved(q[..., dn:], pos, 100.0, 4)
    uk, uv = W["a.uk"].reshape(H, dn, R), W["a.uv"].reshape(H, dv, R)
    for t in range(9):
        qa = np.concatenate([np.einsum("hd,hdr->hr", q[t, :, :dn], uk), qr[t]], axis=1)
        lat = plain.attend_latent(qa, np.concatenate([c, kr], axis=1), W["a.sink"], 0.4, t + 1)[:, :R]
        assert np.allclose(np.einsum("hr,hvr->hv", lat, uv), want[t])
