"""Host-side checks of the Kibotar configuration reader and of the host arithmetic beside its kernels: sizes and constants
come from the configuration alone, the layer order with its repeated range, the rank of the decay projection from the
checkpoint, the rotation's frequency rule, and the cache rows of averaged blocks."""
import copy
import math

import pytest
import torch

import kibotar_plain as P
from mistralrs_b200 import kibotar, mixers, registry, seq_ops


def attention(**kw):
    m = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.3, "mask": {"size": 5, "pool": 3},
         "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 8}}}
    m.update(kw)
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": 9}}


def latent():
    return {"type": "latent_attention", "mixer": {"heads": 3, "dim": 4, "vdim": 5, "kv_rank": 7, "scale": 0.5}, "mlp": None}


def gla():
    return {"type": "gla", "mixer": {"heads": 2, "dim": 6, "vdim": 3, "tau": 4.0}, "mlp": {"kind": "dense", "ff": 11}}


def cfg(layers, **kw):
    cj = {"architecture": "Kibotar", "vocab": 19, "width": 14, "norm": {"eps": 1e-5},
          "embedding": {"scale": 3.0, "bigram": {"buckets": 11, "mul_prev": 5, "mul_cur": 3}}, "layers": layers}
    cj.update(kw)
    return cj


def test_shapes_follow_the_configuration():
    c = kibotar.KibotarConfig(cfg([attention(), latent(), gla()], loop={"start": 1, "stop": 3, "times": 2}))
    s = c.tensor_shapes()
    assert (c.embedding_scale, c.bigram, c.eps) == (3.0, (11, 5, 3), 1e-5)
    assert s["embed"] == (19, 14) and s["bigram"] == (12, 14) and s["loop.step"] == (2, 14) and "head" not in s
    assert s["l0.mix.q"] == (32, 14) and s["l0.mix.k"] == (16, 14) and s["l0.mix.v"] == (12, 14) and s["l0.mix.g"] == (24, 14)
    assert s["l0.mix.talk"] == (4, 4) and s["l0.mix.o.b"] == (14,) and s["l0.mix.o"] == (14, 24)
    assert s["l1.mix.dkv"] == (7, 14) and s["l1.mix.uk"] == (12, 7) and s["l1.mix.uv"] == (15, 7) and s["l1.mix.g"] == (3, 14)
    assert s["l2.mix.a1"] == (None, 14) and s["l2.mix.a2"] == (12, None) and s["l2.mix.norm"] == (3,)
    assert "l1.norm2" not in s and s["l2.norm2b"] == (14,) and all(s[f"l{i}.shift"] == (14,) for i in range(3))
    t = kibotar.random_tensors(c, 1, decay_rank=5)
    assert set(t) == set(s) and t["l2.mix.a1"].shape == (5, 14) and t["l2.mix.a2"].shape == (12, 5)
    assert c.runs() == [(0, None), (1, 0), (2, None), (1, 1), (2, None)] == P.layer_runs(c.raw)


def test_no_repeated_range_and_a_single_pass():
    assert kibotar.KibotarConfig(cfg([gla(), latent()])).runs() == [(0, None), (1, None)]
    once = kibotar.KibotarConfig(cfg([gla(), latent()], loop={"start": 1, "stop": 2, "times": 1}))
    assert once.runs() == [(0, None), (1, 0)] and once.tensor_shapes()["loop.step"] == (1, 14)
    for bad in ({"start": 1, "stop": 1, "times": 2}, {"start": 0, "stop": 3, "times": 2}, {"start": 0, "stop": 1, "times": 0}):
        with pytest.raises(ValueError):
            kibotar.KibotarConfig(cfg([gla(), latent()], loop=bad))


def test_unknown_branches_are_refused():
    bad = cfg([gla()])
    bad["layers"][0]["type"] = "other"
    with pytest.raises(NotImplementedError):
        kibotar.KibotarConfig(bad)
    bad = cfg([gla()])
    bad["layers"][0]["mlp"]["kind"] = "moe"
    with pytest.raises(NotImplementedError):
        kibotar.KibotarConfig(bad)
    with pytest.raises(ValueError):
        kibotar.KibotarConfig(cfg([attention(heads=3)]))
    with pytest.raises(ValueError):
        kibotar.KibotarConfig(cfg([attention(mask={"pool": 4})]))
    with pytest.raises(ValueError):
        kibotar.KibotarConfig(cfg([gla()], architecture="Fosulix"))
    assert "Kibotar" in registry.registered()


@pytest.mark.parametrize("scaling", [None, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}, {"factor": 3.0, "low": 0.5, "high": 8.0, "original": 200}])
def test_rotation_frequencies(scaling):
    rot = {"base": 5000.0, "dims": 24}
    if scaling:
        rot["scaling"] = scaling
    r = mixers.Rotation(24, 5000.0, scaling, torch.device("cpu"))
    assert r.mag == 1.0 and (r.freq - P.rotation_frequencies(rot)).abs().max() < 1e-15
    other = mixers.Rotation(24, 5000.0, {"factor": 8.0, "original": 64, "fast": 4.0, "slow": 1.0}, torch.device("cpu"))      # the ramp-by-index rule stays
    assert other.mag == pytest.approx(0.1 * math.log(8.0) + 1.0) and other.key != r.key


@pytest.mark.parametrize("page_size,pool", [(16, 8), (16, 5), (4, 6), (8, 8), (16, 1), (4, 64)])
def test_rows_of_averaged_blocks_never_collide(page_size, pool):
    """The row of block b: its page's share of rows plus its rank among the blocks that start in that page.  No two blocks
    of one sequence share a row, and the rows stay inside what `pool_rows` reserves."""
    n_pages = 9
    per_page = -(-page_size // pool)
    assert seq_ops.pool_rows(n_pages * page_size, page_size, pool) == n_pages * per_page
    table = [7, 2, 5, 0, 8, 1, 3, 6, 4]
    rows = set()
    for b in range((n_pages * page_size) // pool):
        page = (b * pool) // page_size
        first = -(-(page * page_size) // pool)
        row = table[page] * per_page + (b - first)
        assert 0 <= b - first < per_page and row not in rows and row < n_pages * per_page
        rows.add(row)
