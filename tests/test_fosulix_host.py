"""Host-side checks of the Fosulix configuration reader: sizes and constants come from the configuration alone, every
branch it names is read, and a layer may only reuse the latent of an earlier layer that forms its own."""
import copy

import pytest

from mistralrs_b200 import fosulix, registry


def latent(kv_from=None, **kw):
    m = {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 12, "q_rank": 10, "kv_rank": 6, "scale": 0.25, "mask": {"size": 5},
         "rot": {"base": 100.0, "dims": 4}}
    m.update(kw)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": None}


def gate():
    return {"type": "hgrn2", "mixer": {"heads": 3, "dim": 4, "vdim": 5},
            "mlp": {"kind": "moe", "expert": {"ff": 7, "limit": 3.0}, "router": {"experts": 4, "top": 2, "scale": 2.0, "groups": {"count": 2, "keep": 1}}}}


def cfg(layers, **kw):
    cj = {"architecture": "Fosulix", "vocab": 19, "width": 14, "norm": {"eps": 1e-5}, "residual_mult": 0.25, "embedding": {"scale": 3.0},
          "canon": {"taps": 4}, "layers": layers}
    cj.update(kw)
    return cj


def test_shapes_follow_the_configuration():
    c = fosulix.FosulixConfig(cfg([latent(), gate(), latent(kv_from=0, heads=3, dim=2)]))
    s = c.tensor_shapes()
    assert (c.residual_mult, c.embedding_scale, c.taps, c.eps) == (0.25, 3.0, 4, 1e-5)
    assert s["embed"] == (19, 14) and "head" not in s                      # the logits reuse the embedding table
    assert s["l0.mix.dkv"] == (6 + 4, 14) and s["l0.mix.uq"] == (2 * (8 + 4), 10) and s["l0.mix.uk"] == (2 * 8, 6) and s["l0.mix.uv"] == (2 * 12, 6)
    assert "l2.mix.dkv" not in s and "l2.mix.dkv.norm" not in s and s["l2.mix.uk"] == (3 * 2, 6)
    assert s["l1.mix.lower"] == (12,) and s["l1.mix.norm"] == (5,) and s["l1.mlp.e3.down"] == (14, 7) and s["l1.mlp.router"] == (4, 14)
    assert [s[f"l{i}.dwa"] for i in range(3)] == [(2,), (3,), (4,)] and s["l1.canon1"] == (14, 4)
    assert "l0.norm2" not in s and "l1.norm2" in s
    t = fosulix.random_tensors(c, 1)
    assert set(t) == set(s) and all(tuple(t[k].shape) == tuple(v) for k, v in s.items())


def test_reuse_must_point_at_an_earlier_owner():
    for bad in ([latent(kv_from=0)], [latent(), latent(kv_from=2), latent()], [gate(), latent(kv_from=0)],
                [latent(), latent(kv_from=0), latent(kv_from=1)], [latent(), latent(kv_from=0, kv_rank=8)], [latent(), latent(kv_from=0, rot_dim=2)]):
        with pytest.raises(ValueError):
            fosulix.FosulixConfig(cfg(copy.deepcopy(bad)))


def test_unknown_branches_are_refused():
    bad = cfg([gate()])
    bad["layers"][0]["type"] = "other"
    with pytest.raises(NotImplementedError):
        fosulix.FosulixConfig(bad)
    bad = cfg([gate()])
    bad["layers"][0]["mlp"]["kind"] = "dense"
    with pytest.raises(NotImplementedError):
        fosulix.FosulixConfig(bad)
    with pytest.raises(ValueError):
        fosulix.FosulixConfig(cfg([gate()], architecture="Kilizen"))
    assert "Fosulix" in registry.registered()
