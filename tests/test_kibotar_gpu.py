"""Kibotar on the step engine against the plain float64 restatement (tests/kibotar_plain.py): every mechanism alone,
then whole prompts, token-by-token decoding, portions of many sizes, mixed batches, reused pages and slots, edges of the
window and of the averaged blocks, far keys, a state carried far, long decoding, and greedy generation through the
scheduler.  Small random configurations made here; f32 mode is held to f32 rounding, bf16 mode to bf16 rounding."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import kibotar_plain as P
from mistralrs_b200 import engine, kibotar, mixers, seq_ops as K

pytestmark = pytest.mark.gpu
F64 = torch.float64

WAVES = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}
DENSE = {"kind": "dense", "ff": 56}


def attn_layer(heads=6, kv_heads=2, dim=24, vdim=40, window=21, pool=4, rot_dims=16, base=10000.0, scaling=WAVES, scale=0.2, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window, "pool": pool},
         "rot": {"base": base, "dims": rot_dims}}
    if scaling:
        m["rot"]["scaling"] = dict(scaling)
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent_layer(heads=4, dim=24, vdim=40, kv_rank=56, scale=0.2, mlp=None):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}, "mlp": mlp}


def gla_layer(heads=3, dim=24, vdim=40, tau=8.0, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp}


def make_cfg(layers, width=72, vocab=131, eps=1e-5, emb=4.0, bigram=(97, 31, 7), loop=None):
    cj = {"architecture": "Kibotar", "vocab": vocab, "width": width, "norm": {"eps": eps},
          "embedding": {"scale": emb, "bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}, "layers": layers}
    if loop:
        cj["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cj


FULL = make_cfg([gla_layer(mlp=DENSE), attn_layer(mlp=DENSE), latent_layer(mlp=None), gla_layer(heads=2, dim=16, vdim=16, tau=2.0, mlp=DENSE),
                 attn_layer(heads=4, kv_heads=4, dim=16, vdim=16, window=33, pool=16, rot_dims=8, scaling=None, base=500.0, mlp=None),
                 latent_layer(heads=2, dim=32, vdim=24, kv_rank=40, scale=0.15, mlp=DENSE)], loop=(1, 4, 3))
SMALL = make_cfg([attn_layer(window=9, pool=3, mlp=DENSE), gla_layer(mlp=None), latent_layer(mlp=DENSE)], emb=1.0, loop=(0, 1, 1))


def build(cj, dtype, device, seed=0, page_size=16, edit=None, decay_rank=8):
    cfg = kibotar.KibotarConfig(copy.deepcopy(cj))
    tensors = kibotar.random_tensors(cfg, seed, decay_rank)
    if edit:
        edit(tensors)
    model = kibotar.KibotarModel(cfg, tensors, device, dtype, page_size=page_size)
    return model, {k: v.to(F64) for k, v in tensors.items()}


def rel_err(got, want):
    """Per row: rms of the difference (mean taken off) over the rms of the wanted logits."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt((want ** 2).mean())


TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}


def assert_close(got, want, dtype, what=""):
    e = rel_err(got, want)
    if dtype == torch.float32:
        assert e.max() < TOL[dtype], (what, float(e.max()), int(e.argmax()))
    else:
        assert (e > TOL[dtype]).sum() <= max(1, 0.03 * e.size) and np.median(e) < TOL[dtype] / 3, (what, float(e.max()), float(np.median(e)))


def replay(eng, prompts, schedule):
    """schedule: steps, each a list of (name, n_tokens).  Returns name -> logits of every position [T, vocab]."""
    live, rows = {}, {k: [] for k in prompts}
    for step in schedule:
        plan, want = [], []
        for name, n in step:
            if name not in live:
                live[name] = eng.new_request([])
            r = live[name]
            at = r.n_computed
            r.tokens.extend(prompts[name][at:at + n])
            plan.append((r, n))
            want.append(list(range(n)))
        lg = eng.execute(plan, want).cpu().numpy()
        at = 0
        for name, n in step:
            rows[name].append(lg[at:at + n])
            at += n
            if live[name].n_computed == len(prompts[name]):
                eng.finish(live.pop(name))
    return {k: np.concatenate(v) for k, v in rows.items() if v}


def tokens(n, vocab, seed):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def close_rows(got, want, tol):
    """Every row within tol; at bf16 tolerances 2 % of the rows may reach three times tol."""
    e = (got - want).norm(dim=-1) / want.norm(dim=-1).mean()
    if tol >= 1e-2:
        assert (e > tol).double().mean() <= 0.02 and e.max() < 3 * tol, (float(e.max()), int(e.argmax()))
    else:
        assert e.max() < tol, (float(e.max()), int(e.argmax()))


# ---- mechanisms alone ------------------------------------------------------------------------------------------------
def seq_batch(device, portions, page_size=16, ids=None):
    """One step of several sequences: portions = [(n_new, past, slot, first_page)]."""
    counts, pasts, slots, tables, slot_map = [], [], [], [], []
    for n, past, slot, first_page in portions:
        pages = list(range(first_page, first_page + -(-(past + n) // page_size)))
        counts.append(n), pasts.append(past), slots.append(slot), tables.append(pages)
        slot_map += [pages[(past + i) // page_size] * page_size + (past + i) % page_size for i in range(n)]
    return engine.StepBatch(device, ids if ids is not None else [0] * sum(counts), counts, pasts, slots, tables, np.asarray(slot_map, dtype=np.int64), [])


def plain_mixer(layer, h, w, eps, p="l0.mix."):
    if layer["type"] == "gla":
        return P.gated_linear_attention(h, w, p, layer["mixer"], eps)
    if layer["type"] == "latent_attention":
        return P.latent_attention(h, w, p, layer["mixer"], eps)
    return P.pooled_window_attention(h, w, p, layer["mixer"])


def mixer_case(cuda, layer, dtype, T, portions, seed=3, edit=None, width=72, h=None, pages=80, page_size=16, first_page=3):
    """Run layer 0's mixer alone over `portions` of one sequence; returns (got [T, W], want [T, W])."""
    cj = make_cfg([layer], width=width)
    model, w = build(cj, dtype, cuda, seed, edit=edit, page_size=page_size)
    if h is None:
        h = torch.randn(T, width, generator=torch.Generator().manual_seed(seed))
    h = h.to(dtype)
    mixer = model.layers[0].mixer
    cache = mixer.alloc_cache(2, page_size * pages, dtype, cuda)
    for c in cache.values():
        c.normal_()                      # whatever an earlier request left: a sequence that starts must not see it
    got, at = [], 0
    for n in portions:
        got.append(mixer.forward(h[at:at + n].to(cuda).contiguous(), seq_batch(cuda, [(n, at, 1, first_page)], page_size), cache).double().cpu())
        at += n
    return torch.cat(got), plain_mixer(layer, h.double(), w, 1e-5)


def test_pair_embedding(cuda):
    """Table row times scale plus the hashed pair row; the previous token crosses portions through a slot that held another
    request's token, and a sequence's first token takes the table's last row."""
    g = torch.Generator().manual_seed(1)
    V, W, buckets, mp, mc = 50, 24, 13, 31, 7
    table, pairs = torch.randn(V, W, generator=g), torch.randn(buckets + 1, W, generator=g)
    a, b = tokens(30, V, 1), tokens(9, V, 2)
    want = {"a": P.embed(a, table.double(), 3.0, pairs.double(), buckets, mp, mc), "b": P.embed(b, table.double(), 3.0, pairs.double(), buckets, mp, mc)}
    state = torch.full((3,), 49, dtype=torch.int32, device=cuda)
    got = {"a": [], "b": []}
    for (na, pa), (nb, pb) in [((1, 0), (2, 0)), ((2, 1), (1, 2)), ((20, 3), (5, 3)), ((7, 23), (1, 8))]:
        ids = a[pa:pa + na] + b[pb:pb + nb]
        batch = seq_batch(cuda, [(na, pa, 2, 1), (nb, pb, 0, 9)], ids=ids)
        out = torch.empty(na + nb, W, device=cuda)
        K.embed_pair(table.to(cuda), pairs.to(cuda), batch.ids, 3.0, buckets, mp, mc, state, batch, out)
        got["a"].append(out[:na].double().cpu()), got["b"].append(out[na:].double().cpu())
    for k in want:
        assert (torch.cat(got[k]) - want[k]).abs().max() < 1e-5
    assert state.tolist() == [b[-1], 49, a[-1]]


def test_token_shift(cuda):
    """h + (h_prev - h) * mu over portions of two sequences side by side; the carried input lives in slots that held other data."""
    g = torch.Generator().manual_seed(2)
    mu = torch.rand(40, generator=g) * 1.4 - 0.2
    shift = mixers.TokenShift(mu.to(cuda))
    state = shift.alloc_cache(3, cuda).normal_()
    a, b = torch.randn(30, 40, generator=g), torch.randn(9, 40, generator=g)
    want = {"a": P.token_shift(a.double(), mu.double()), "b": P.token_shift(b.double(), mu.double())}
    got = {"a": [], "b": []}
    for (na, pa), (nb, pb) in [((1, 0), (2, 0)), ((2, 1), (1, 2)), ((20, 3), (5, 3)), ((7, 23), (1, 8))]:
        x = torch.cat([a[pa:pa + na], b[pb:pb + nb]]).to(cuda)
        y = shift.forward(x, seq_batch(cuda, [(na, pa, 2, 1), (nb, pb, 0, 9)]), state).double().cpu()
        got["a"].append(y[:na]), got["b"].append(y[na:])
    for k in want:
        assert (torch.cat(got[k]) - want[k]).abs().max() < 1e-5


@pytest.mark.parametrize("width", [64, 45])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_residual_step_with_norms_on_both_sides(cuda, width, dtype):
    """x + rms_norm(y) * w_post + a vector, then the next norm, in place — against the same in float64."""
    g = torch.Generator().manual_seed(width)
    T = 19
    src, y = torch.randn(T, width, generator=g), (3.0 * torch.randn(T, width, generator=g)).to(dtype)
    pw, nw, vec = torch.randn(width, generator=g), torch.randn(width, generator=g), torch.randn(width, generator=g)
    x = src.to(cuda)
    h = K.rms_residual(x, y.to(cuda), dst=x, post_w=pw.to(cuda), add_vec=vec.to(cuda), next_w=nw.to(cuda), eps=1e-5)
    new = src.double() + P.unit_rms(y.double(), 1e-5) * pw.double() + vec.double()
    assert (x.double().cpu() - new).abs().max() < 1e-5
    close_rows(h.double().cpu(), P.unit_rms(new, 1e-5) * nw.double(), 1e-5 if dtype == torch.float32 else 1e-2)
    x = src.to(cuda)                                          # no sublayer output: only the vector and the norm
    h = K.rms_residual(x, dst=x, add_vec=vec.to(cuda), next_w=nw.to(cuda), eps=1e-5, dtype=dtype)
    assert (x.double().cpu() - (src.double() + vec.double())).abs().max() < 1e-6
    close_rows(h.double().cpu(), P.unit_rms(src.double() + vec.double(), 1e-5) * nw.double(), 1e-5 if dtype == torch.float32 else 1e-2)
    x = src.to(cuda)                                          # the last step of a model: no next norm
    assert K.rms_residual(x, y.to(cuda), dst=x, post_w=pw.to(cuda), eps=1e-5) is None
    assert (x.double().cpu() - (src.double() + P.unit_rms(y.double(), 1e-5) * pw.double())).abs().max() < 1e-5


def test_power_gate(cuda):
    """sigmoid(z + b)^(1 / tau) in f32 for pre-activations from deep saturation to deep cut-off."""
    z = torch.linspace(-90.0, 90.0, 181 * 3).view(3, 181)
    b = torch.linspace(-1.0, 1.0, 181)
    for tau in (1.0, 16.0, 0.5):
        got = K.power_gate(z.to(cuda), 0, 181, b.to(cuda), 1.0 / tau).double().cpu()
        want = P.sigmoid(z.double() + b.double()) ** (1.0 / tau)
        assert (got - want).abs().max() < 2e-6 and ((got - want).abs() / want.clamp_min(1e-30))[want > 1e-30].max() < 1e-4


def test_rotation_frequencies_by_wavelength(cuda):
    """Kept, blended and slowed frequencies all occur; the table turns halves."""
    rot = {"base": 10000.0, "dims": 32, "scaling": WAVES}
    want = P.rotation_frequencies(rot)
    plain = P.rotation_frequencies({"base": 10000.0, "dims": 32})
    ratio = (want / plain)
    assert (ratio == 1.0).any() and (ratio == 0.25).any() and ((ratio > 0.25) & (ratio < 1.0)).any()
    r = mixers.Rotation(32, 10000.0, WAVES, cuda)
    assert (r.freq.cpu() - want).abs().max() < 1e-15 and r.mag == 1.0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("portions", [[150], [1] * 40, [7, 2, 33, 1, 64, 2, 41]])
@pytest.mark.parametrize("layer", [attn_layer(), latent_layer(), gla_layer()], ids=["attention", "latent", "gla"])
def test_mixers(cuda, layer, dtype, tol, portions):
    got, want = mixer_case(cuda, layer, dtype, sum(portions), portions)
    close_rows(got, want, tol)


@pytest.mark.parametrize("layer", [attn_layer(heads=1, kv_heads=1, dim=8, vdim=8, window=1, pool=1, rot_dims=2),
                                   attn_layer(heads=5, kv_heads=5, dim=7, vdim=9, window=200, pool=5, rot_dims=6, scaling=None),
                                   attn_layer(heads=8, kv_heads=1, dim=64, vdim=64, window=16, pool=16, rot_dims=64),
                                   attn_layer(heads=4, kv_heads=2, dim=16, vdim=136, window=7, pool=3, rot_dims=16, scaling={"factor": 3.0, "low": 0.5, "high": 2.0, "original": 16}),
                                   attn_layer(heads=12, kv_heads=4, dim=32, vdim=16, window=30, pool=7, rot_dims=8, base=50.0),
                                   attn_layer(heads=2, kv_heads=2, dim=16, vdim=16, window=5, pool=40, rot_dims=4),
                                   attn_layer(heads=8, kv_heads=8, dim=16, vdim=136, window=9, pool=2, rot_dims=8),
                                   attn_layer(heads=4, kv_heads=2, dim=16, vdim=600, window=9, pool=2, rot_dims=8),
                                   attn_layer(heads=4, kv_heads=2, dim=16, vdim=24, window=0, pool=0, rot_dims=8)])
def test_attention_other_sizes(cuda, layer):
    """One or all heads sharing keys, full / partial rotation, key size != value size, blocks of 1, blocks that do not divide a
    page, blocks larger than a page, a block larger than the window, a window wider than the sequence, value heads that together
    are wider than one launch of the kernel takes, no window at all."""
    got, want = mixer_case(cuda, layer, torch.float32, 100, [25, 1, 1, 3, 30, 40], width=48)
    close_rows(got, want, 3e-5)


TC_LAYERS = [attn_layer(heads=4, kv_heads=2, dim=64, vdim=64, window=70, pool=8, rot_dims=32),
             attn_layer(heads=3, kv_heads=1, dim=128, vdim=128, window=64, pool=16, rot_dims=64),
             attn_layer(heads=8, kv_heads=4, dim=64, vdim=64, window=200, pool=5, rot_dims=64, scaling=None),
             attn_layer(heads=2, kv_heads=2, dim=64, vdim=64, window=33, pool=1, rot_dims=16)]


@pytest.mark.parametrize("layer", TC_LAYERS)
@pytest.mark.parametrize("portions", [[300], [70, 33, 1, 196], [31, 269]])
def test_attention_tensor_core_kernel(cuda, layer, portions):
    """bf16 portions of 32 tokens or more run on the tensor-core prompt kernel, once per value head: fresh and continued
    portions, windows and averaged blocks inside and across its key tiles, one / some / all heads sharing a value head."""
    got, want = mixer_case(cuda, layer, torch.bfloat16, sum(portions), portions)
    close_rows(got, want, 3e-2)


def test_averaged_blocks_without_head_mixing(cuda):
    """The mechanisms are separate: a layer with averaged blocks but no mixing matrix (identity in the plain model), on the
    (token, head) kernel in f32 and on tensor cores in bf16."""
    for dtype, tol, layer in ((torch.float32, 3e-5, attn_layer(pool=4)), (torch.bfloat16, 3e-2, TC_LAYERS[0])):
        cj = make_cfg([layer])
        model, w = build(cj, dtype, cuda, 3)
        mixer = model.layers[0].mixer
        mixer.attn.talk = None
        w["l0.mix.talk"] = torch.eye(layer["mixer"]["heads"], dtype=F64)
        h = torch.randn(150, 72, generator=torch.Generator().manual_seed(3)).to(dtype)
        cache = mixer.alloc_cache(1, 16 * 20, dtype, cuda)
        got, at = [], 0
        for n in (90, 1, 59):
            got.append(mixer.forward(h[at:at + n].to(cuda).contiguous(), seq_batch(cuda, [(n, at, 0, 2)]), cache).double().cpu())
            at += n
        close_rows(torch.cat(got), plain_mixer(layer, h.double(), w, 1e-5), tol)


def test_tensor_core_kernel_takes_several_sequences(cuda):
    """Two sequences start in one step beside a long portion that continues a third and a single decoded token of a fourth."""
    layer = TC_LAYERS[0]
    cj = make_cfg([layer], width=64)
    model, w = build(cj, torch.bfloat16, cuda, 7)
    mixer = model.layers[0].mixer
    cache = mixer.alloc_cache(4, 16 * 60, torch.bfloat16, cuda)
    g = torch.Generator().manual_seed(7)
    hs = [torch.randn(n, 64, generator=g).to(torch.bfloat16) for n in (150, 33, 130, 12)]
    mixer.forward(torch.cat([hs[2][:90], hs[3][:11]]).to(cuda).contiguous(), seq_batch(cuda, [(90, 0, 2, 30), (11, 0, 3, 40)]), cache)
    b = seq_batch(cuda, [(150, 0, 0, 1), (40, 90, 2, 30), (1, 11, 3, 40), (33, 0, 1, 12)])
    assert len(b.long) == 3 and b.short_tok.numel() == 1
    got = mixer.forward(torch.cat([hs[0], hs[2][90:], hs[3][11:], hs[1]]).to(cuda).contiguous(), b, cache).double().cpu()
    want = [plain_mixer(layer, h.double(), w, 1e-5) for h in hs]
    close_rows(got, torch.cat([want[0], want[2][90:], want[3][11:], want[1]]), 3e-2)


@pytest.mark.parametrize("page_size,pool", [(4, 3), (4, 8), (16, 5), (32, 12), (8, 8)])
def test_averaged_blocks_across_pages(cuda, page_size, pool):
    """Blocks that straddle pages, span several pages, or fill one exactly; the pages of the sequence are not the first of the pool."""
    layer = attn_layer(heads=4, kv_heads=2, dim=16, vdim=24, window=11, pool=pool, rot_dims=8)
    got, want = mixer_case(cuda, layer, torch.float32, 90, [13, 1, 1, 30, 2, 43], width=48, page_size=page_size, pages=40, first_page=5)
    close_rows(got, want, 3e-5)


@pytest.mark.parametrize("layer", [latent_layer(heads=1, dim=8, vdim=8, kv_rank=8), latent_layer(heads=5, dim=7, vdim=9, kv_rank=11),
                                   latent_layer(heads=16, dim=16, vdim=136, kv_rank=264), latent_layer(heads=3, dim=40, vdim=8, kv_rank=520)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
def test_latent_other_sizes(cuda, layer, dtype, tol):
    got, want = mixer_case(cuda, layer, dtype, 70, [25, 1, 1, 3, 40], width=48)
    close_rows(got, want, tol)


@pytest.mark.parametrize("layer", [latent_layer(heads=3, dim=64, vdim=64, kv_rank=40), latent_layer(heads=2, dim=128, vdim=128, kv_rank=264)])
@pytest.mark.parametrize("portions", [[300], [300, 1, 1, 40], [257, 43]])
def test_latent_whole_prompt_is_decompressed(cuda, layer, portions, monkeypatch):
    """A step in which every sequence starts with a long portion decompresses keys and values for that step and runs the plain
    tensor-core kernel over them; what follows (decoded tokens, later portions) reads the cached latents in the absorbed form."""
    seen = []
    real = K.dense_prompt_attention
    monkeypatch.setattr(K, "dense_prompt_attention", lambda *a, **k: (seen.append(1), real(*a, **k))[1])
    got, want = mixer_case(cuda, layer, torch.bfloat16, sum(portions), portions)
    assert len(seen) == 1
    close_rows(got, want, 3e-2)


def test_latent_decompressed_for_two_prompts_at_once(cuda, monkeypatch):
    layer = latent_layer(heads=3, dim=64, vdim=64, kv_rank=40)
    cj = make_cfg([layer], width=64)
    model, w = build(cj, torch.bfloat16, cuda, 7)
    mixer = model.layers[0].mixer
    cache = mixer.alloc_cache(2, 16 * 40, torch.bfloat16, cuda)
    g = torch.Generator().manual_seed(7)
    hs = [torch.randn(n, 64, generator=g).to(torch.bfloat16) for n in (200, 90)]
    b = seq_batch(cuda, [(200, 0, 0, 1), (90, 0, 1, 20)])
    assert mixer.decompresses(torch.cat(hs), b)
    got = mixer.forward(torch.cat(hs).to(cuda).contiguous(), b, cache).double().cpu()
    close_rows(got, torch.cat([plain_mixer(layer, h.double(), w, 1e-5) for h in hs]), 3e-2)
    b2 = seq_batch(cuda, [(200, 0, 0, 1), (1, 90, 1, 20)])          # a decoded token beside a prompt: the absorbed form for both
    assert not mixer.decompresses(torch.cat(hs), b2)


@pytest.mark.parametrize("layer", [gla_layer(heads=1, dim=7, vdim=5, tau=1.0), gla_layer(heads=5, dim=136, vdim=24, tau=3.0),
                                   gla_layer(heads=2, dim=16, vdim=200, tau=64.0), gla_layer(heads=2, dim=600, vdim=8, tau=16.0)])
def test_gla_other_sizes(cuda, layer):
    got, want = mixer_case(cuda, layer, torch.float32, 60, [25, 1, 1, 3, 30], width=48)
    close_rows(got, want, 3e-5)


def test_gla_scan_in_segments(cuda, monkeypatch):
    """Long portions are scanned as segments side by side and chained: forced onto a short one, cut in the middle of a segment."""
    monkeypatch.setattr(K, "SCAN_SEGMENT_MIN_TOKENS", 64)
    monkeypatch.setattr(K, "SCAN_SEGMENT", 32)
    got, want = mixer_case(cuda, gla_layer(), torch.float32, 250, [100, 1, 149])
    close_rows(got, want, 3e-5)


def test_gla_first_token_survives_far(cuda):
    """With decays at one (a large bias) the first token's value is still read after 300 steps; the plain model without the first
    token differs."""
    layer = gla_layer(heads=2, dim=16, vdim=16, tau=16.0)

    def edit(t):
        t["l0.mix.a2.b"].fill_(30.0)
        t["l0.mix.a2"].zero_()
    T = 300
    h = 0.05 * torch.randn(T, 48, generator=torch.Generator().manual_seed(4))
    h[0] *= 60.0
    got, want = mixer_case(cuda, layer, torch.float32, T, [280] + [1] * 20, edit=edit, width=48, h=h)
    close_rows(got, want, 3e-5)
    cj = make_cfg([layer], width=48)
    _, w = build(cj, torch.float32, cuda, 3, edit=edit)
    h2 = h.clone()
    h2[0] = 0.0
    assert (plain_mixer(layer, h2.double(), w, 1e-5)[-1] - want[-1]).norm() > 0.2 * want[-1].norm()


def test_decay_shows(cuda):
    """A temperature of 1 forgets quickly, a large one slowly: the two differ, and each matches its plain counterpart."""
    outs = []
    for tau in (1.0, 32.0):
        got, want = mixer_case(cuda, gla_layer(tau=tau), torch.float32, 40, [40])
        close_rows(got, want, 3e-5)
        outs.append(want)
    assert (outs[0] - outs[1]).norm() > 0.1 * outs[1].norm()


def pointed_attention_edit(width, dk, dv, heads, kv_heads, rot=False):
    """Projections under which every head's query and every key head's key are the input's first dk entries and the values the
    next dv entries: a query scores high with exactly the keys whose input shares its direction there.  No biases, gates open
    wide, rotation left to the configuration."""
    def edit(t):
        eye = lambda r, c, off=0: torch.cat([torch.zeros(r, off), torch.eye(r, c - off)], dim=1)
        t["l0.mix.q"].copy_(eye(dk, width).repeat(heads, 1).to(torch.bfloat16))
        t["l0.mix.k"].copy_(eye(dk, width).repeat(kv_heads, 1).to(torch.bfloat16))
        t["l0.mix.v"].copy_(eye(dv, width, dk).repeat(kv_heads, 1).to(torch.bfloat16))
        for b in ("q.b", "k.b", "v.b", "o.b"):
            t["l0.mix." + b].zero_()
        t["l0.mix.g"].zero_()
        t["l0.mix.g"][:, -1] = 8.0
    return edit


def pointed_inputs(T, width, dk, target, seed, gain=3.0):
    """Random inputs whose first dk entries are small except in the last token and in `target`, which share a direction
    there (the target `gain` times as long — a target that is seen as one of a block's average needs the block's size more)
    and differ elsewhere; the last entry is one everywhere (it opens the gates)."""
    query = T - 1
    h = torch.randn(T, width, generator=torch.Generator().manual_seed(seed))
    h[:, :dk] *= 0.3
    h[query, :dk] *= 10.0
    h[target, :dk] = gain * h[query, :dk]
    h[:, -1] = 1.0
    return h


# the same edges on the (token, head) kernel in f32 and, with heads of 64, on the tensor-core prompt kernel in bf16
EDGE_KINDS = [(torch.float32, 3e-5, 16, 24, 64), (torch.bfloat16, 3e-2, 64, 64, 136)]


@pytest.mark.parametrize("distance", [-2, -1, 0, 1])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("dtype,tol,dk,dv,width", EDGE_KINDS, ids=["f32", "bf16-tensor-cores"])
def test_window_edge_shows(cuda, distance, decoded, dtype, tol, dk, dv, width):
    """One earlier token shares the last query's direction under a large score scale; it sits around the window's far edge, and
    one step outside it is gone (its block is not yet whole).  The blocks are long, so no averaged entry hides the edge."""
    window, T = 24, 120
    target = T - 1 - (window - 1) - distance                   # distance <= 0: in sight
    layer = attn_layer(heads=4, kv_heads=2, dim=dk, vdim=dv, window=window, pool=64, rot_dims=0, scale=16.0 / dk)
    layer["mixer"].pop("rot")
    h = pointed_inputs(T, width, dk, target, 9).to(dtype).float()
    cuts = [T - 3, 1, 1, 1] if decoded else [T]
    got, want = mixer_case(cuda, layer, dtype, T, cuts, seed=9, edit=pointed_attention_edit(width, dk, dv, 4, 2), width=width, h=h)
    close_rows(got, want, tol)
    cj = make_cfg([layer], width=width)
    _, w = build(cj, torch.float32, cuda, 9, edit=pointed_attention_edit(width, dk, dv, 4, 2))
    other = copy.deepcopy(layer)
    other["mixer"]["mask"]["size"] = window + distance if distance > 0 else window - 1 + distance
    assert (plain_mixer(other, h.double(), w, 1e-5)[-1] - want[-1]).norm() > 0.2 * want[-1].norm()


@pytest.mark.parametrize("missing", [0, 1])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("pool", [4, 6])
@pytest.mark.parametrize("dtype,tol,dk,dv,width", EDGE_KINDS, ids=["f32", "bf16-tensor-cores"])
def test_block_edge_shows(cuda, pool, missing, decoded, dtype, tol, dk, dv, width):
    """The matching token lies in the newest block before the window.  missing 0: the block's last position has just left the
    window, so its average is seen; missing 1: one of its positions is still inside the window's reach of exclusion — the
    block is not whole yet and the token is seen neither singly nor averaged."""
    window = 10
    nb = 7
    T = nb * pool + window - missing                            # the last query, position T - 1, sees a block that ends at or before T - 1 - window
    target = nb * pool - pool + 1                               # inside block nb - 1
    layer = attn_layer(heads=4, kv_heads=2, dim=dk, vdim=dv, window=window, pool=pool, rot_dims=0, scale=16.0 / dk)
    layer["mixer"].pop("rot")
    h = pointed_inputs(T, width, dk, target, 5, gain=3.0 * pool).to(dtype).float()
    cuts = [T - 3, 1, 1, 1] if decoded else [T]
    got, want = mixer_case(cuda, layer, dtype, T, cuts, seed=5, edit=pointed_attention_edit(width, dk, dv, 4, 2), width=width, h=h)
    close_rows(got, want, tol)
    seen_blocks, lo = P.pooled_window_keys(T - 1, window, pool)
    assert seen_blocks == (nb if missing == 0 else nb - 1) and lo > target
    cj = make_cfg([layer], width=width)
    _, w = build(cj, torch.float32, cuda, 5, edit=pointed_attention_edit(width, dk, dv, 4, 2))
    other = copy.deepcopy(layer)
    other["mixer"]["mask"]["size"] = window + (1 if missing == 0 else -1)       # one wider hides the block, one narrower shows it
    assert (plain_mixer(other, h.double(), w, 1e-5)[-1] - want[-1]).norm() > 0.2 * want[-1].norm()


@pytest.mark.parametrize("target", [0, 15, 16, 17, 333])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("kind", ["attention", "latent"])
def test_far_key_among_hundreds(cuda, kind, target, decoded):
    """One matching key far back among 700: through an averaged block for the windowed attention, singly for the latent one."""
    T, dk = 700, 16
    h = pointed_inputs(T, 64, dk, target, 13, gain=24.0 if kind == "attention" else 3.0)
    cuts = [T - 2, 1, 1] if decoded else [T]
    if kind == "attention":
        layer = attn_layer(heads=4, kv_heads=2, dim=dk, vdim=24, window=40, pool=8, rot_dims=0, scale=1.0)
        layer["mixer"].pop("rot")
        edit = pointed_attention_edit(64, dk, 24, 4, 2)
    else:
        layer = latent_layer(heads=2, dim=dk, vdim=24, kv_rank=32, scale=1.0)

        def edit(t):
            t["l0.mix.dkv"].copy_(torch.eye(32, 64).to(torch.bfloat16))
            t["l0.mix.dkv.norm"].fill_(1.0)
            t["l0.mix.q"].copy_(torch.eye(dk, 64).repeat(2, 1).to(torch.bfloat16))
            t["l0.mix.uk"].copy_(torch.eye(dk, 32).repeat(2, 1).to(torch.bfloat16))
            later = torch.zeros(24, 32)
            later[:dk, dk:2 * dk] = torch.eye(dk)
            t["l0.mix.uv"].copy_(later.repeat(2, 1).to(torch.bfloat16))
    got, want = mixer_case(cuda, layer, torch.float32, T, cuts, seed=13, edit=edit, width=64, h=h, pages=50)
    close_rows(got[-3:], want[-3:], 3e-5)
    h2 = h.clone()
    h2[target, :dk] = 0.0
    cj = make_cfg([layer], width=64)
    _, w = build(cj, torch.float32, cuda, 13, edit=edit)
    assert (plain_mixer(layer, h2.double(), w, 1e-5)[-1] - want[-1]).norm() > 0.1 * want[-1].norm()


def test_one_in_the_denominator_shows(cuda):
    """Scores far below zero: the added one takes most of the mass and the output shrinks; a softmax without it would not."""
    layer = attn_layer(heads=4, kv_heads=2, dim=16, vdim=24, window=12, pool=4, rot_dims=0, scale=-0.2)
    layer["mixer"].pop("rot")
    h = torch.randn(50, 72, generator=torch.Generator().manual_seed(3))
    h[:, :16] = 1.0 + torch.rand(50, 16, generator=torch.Generator().manual_seed(4))        # every query . key is positive: every score negative
    h[:, -1] = 1.0
    got, want = mixer_case(cuda, layer, torch.float32, 50, [30, 1, 19], edit=pointed_attention_edit(72, 16, 24, 4, 2), h=h)
    close_rows(got, want, 3e-5)
    mild = copy.deepcopy(layer)
    mild["mixer"]["scale"] = -0.001
    _, want_mild = mixer_case(cuda, mild, torch.float32, 50, [50], edit=pointed_attention_edit(72, 16, 24, 4, 2), h=h)
    assert want[5:].norm() < 0.2 * want_mild[5:].norm()


def test_head_mixing_shows(cuda):
    """The mixing matrix is far from the identity and heads share value heads in groups: the plain model with an identity differs."""
    layer = attn_layer(heads=6, kv_heads=3, dim=16, vdim=24, window=12, pool=4)

    def edit(t):
        t["l0.mix.talk"].copy_(torch.randn(6, 6, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16))
    got, want = mixer_case(cuda, layer, torch.float32, 60, [33, 1, 1, 25], edit=edit)
    close_rows(got, want, 3e-5)
    cj = make_cfg([layer])
    _, w = build(cj, torch.float32, cuda, 3, edit=edit)
    w["l0.mix.talk"] = torch.eye(6, dtype=F64)
    h = torch.randn(60, 72, generator=torch.Generator().manual_seed(3)).double()
    assert (plain_mixer(layer, h, w, 1e-5) - want).norm() > 0.3 * want.norm()


def test_rotation_turns_halves(cuda):
    """Only rotation decides: keys equal at every position, scores differ through the angle alone; partial rotation."""
    layer = attn_layer(heads=2, kv_heads=2, dim=16, vdim=24, window=64, pool=64, rot_dims=12, base=30.0, scaling=None, scale=2.0)
    T = 50
    h = torch.randn(1, 72, generator=torch.Generator().manual_seed(6)).repeat(T, 1)
    h[:, 16:] = torch.randn(T, 56, generator=torch.Generator().manual_seed(7))               # equal keys, different values
    got, want = mixer_case(cuda, layer, torch.float32, T, [20, 1, 29], edit=pointed_attention_edit(72, 16, 24, 2, 2), h=h)
    close_rows(got, want, 3e-5)
    flat = copy.deepcopy(layer)
    flat["mixer"].pop("rot")
    _, unrotated = mixer_case(cuda, flat, torch.float32, T, [T], edit=pointed_attention_edit(72, 16, 24, 2, 2), h=h)
    assert (unrotated - want).norm() > 0.05 * want.norm()


def test_dense_feed_forward(cuda):
    cj = make_cfg([gla_layer(mlp=DENSE)])
    model, w = build(cj, torch.float32, cuda, 2)
    h = torch.randn(21, 72, generator=torch.Generator().manual_seed(2))
    close_rows(model.layers[0].mlp.forward(h.to(cuda)).double().cpu(), P.dense_ff(h.double(), w, "l0.mlp."), 2e-5)


# ---- the model on the engine ----------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def full32(cuda):
    model, w = build(FULL, torch.float32, cuda, 11)
    prompts = {"a": tokens(150, 131, 1), "b": tokens(37, 131, 2), "c": tokens(2, 131, 3), "d": tokens(75, 131, 4), "e": tokens(1, 131, 5)}
    want = {k: P.forward(FULL, w, v).numpy() for k, v in prompts.items()}
    return model, prompts, want


def test_layer_order(cuda):
    cfg = kibotar.KibotarConfig(copy.deepcopy(FULL))
    assert cfg.runs() == [(0, None), (1, 0), (2, None), (3, None), (1, 1), (2, None), (3, None), (1, 2), (2, None), (3, None), (4, None), (5, None)]
    assert cfg.runs() == P.layer_runs(FULL)
    assert kibotar.KibotarConfig(copy.deepcopy(SMALL)).runs() == [(0, 0), (1, None), (2, None)]
    plain = copy.deepcopy(SMALL)
    plain.pop("loop")
    assert kibotar.KibotarConfig(plain).runs() == [(0, None), (1, None), (2, None)]


def test_whole_prompts_and_layers(cuda, full32):
    model, prompts, want = full32
    eng = engine.Engine(model, max_tokens=160, max_seqs=1)
    for name in prompts:
        got = replay(eng, prompts, [[(name, len(prompts[name]))]])[name]
        assert_close(got, want[name], torch.float32, name)
    _, w = build(FULL, torch.float32, cuda, 11)
    layers = []
    P.forward(FULL, w, prompts["b"], lambda r, x: layers.append(x.clone()))
    seen = {}
    r = eng.new_request(prompts["b"])
    hooked = eng.execute([(r, 37)], after_layer=lambda i, x: seen.__setitem__(i, x.double().cpu())).cpu().numpy()
    eng.finish(r)
    assert len(seen) == len(layers) == 12
    for i in range(len(layers)):
        assert (seen[i] - layers[i]).abs().max() < 2e-4 * layers[i].abs().max(), i
    assert_close(hooked, want["b"][-1:], torch.float32)


def test_decode_token_by_token_equals_prefill(cuda, full32):
    model, prompts, want = full32
    eng = engine.Engine(model, max_tokens=160, max_seqs=1)
    got = replay(eng, prompts, [[("b", 1)] for _ in range(37)])["b"]
    assert_close(got, want["b"], torch.float32)
    got = replay(eng, prompts, [[("a", 60)]] + [[("a", 1)] for _ in range(90)])["a"]      # long decoding across windows, blocks and pages
    assert_close(got, want["a"], torch.float32)


@pytest.mark.parametrize("sizes", [[2] * 75, [3, 16, 1, 15, 17, 2, 32, 31, 2, 2, 29], [149, 1], [16] * 9 + [6]])
def test_portions(cuda, full32, sizes):
    model, prompts, want = full32
    assert sum(sizes) == 150
    eng = engine.Engine(model, max_tokens=160, max_seqs=1)
    got = replay(eng, prompts, [[("a", n)] for n in sizes])["a"]
    assert_close(got, want["a"], torch.float32)


def test_mixed_batches_and_reuse(cuda, full32):
    """Unequal requests side by side, portions beside single tokens; the pools are too small for all of them at once, so
    pages and state slots of finished requests are taken again (by requests that must not see what was left there)."""
    model, prompts, want = full32
    eng = engine.Engine(model, max_tokens=16 * 16, max_seqs=3)
    schedule = [[("a", 40), ("b", 30)], [("a", 1), ("b", 7), ("c", 2)], [("a", 60), ("d", 5)], [("d", 1), ("a", 1)], [("d", 69), ("a", 48), ("e", 1)]]
    got = replay(eng, prompts, schedule)
    for name in prompts:
        assert_close(got[name], want[name], torch.float32, name)
    assert eng.slots.num_free() == 3 and eng.pages.num_free_blocks() == 16
    again = replay(eng, prompts, [[("d", 75), ("b", 37), ("c", 2)], [("a", 100)], [("a", 50)]])    # every slot and page has been used before
    for name in ("a", "b", "d"):
        assert_close(again[name], want[name], torch.float32, name)


def test_a_request_may_sit_out_a_step(cuda, full32):
    model, prompts, want = full32
    eng = engine.Engine(model, max_tokens=16 * 16, max_seqs=2)
    got = replay(eng, prompts, [[("b", 20)], [("d", 30)], [("d", 1)], [("b", 2), ("d", 2)], [("d", 42)], [("b", 15)]])
    for name in ("b", "d"):
        assert_close(got[name], want[name], torch.float32, name)


def test_batch_of_decodes_matches_each_alone(cuda, full32):
    """Also the captured-graph path: from its second occurrence a batch of single tokens replays a CUDA graph."""
    model, prompts, want = full32
    eng = engine.Engine(model, max_tokens=16 * 20, max_seqs=4)
    schedule = [[("a", 120), ("b", 17), ("d", 55)]] + [[("a", 1), ("b", 1), ("d", 1)] for _ in range(20)]
    got = replay(eng, prompts, schedule)
    assert_close(got["a"], want["a"][:140], torch.float32)
    assert_close(got["b"], want["b"], torch.float32)
    assert_close(got["d"], want["d"], torch.float32)
    assert 3 in eng._graphs or not eng.decode_graphs


@pytest.mark.parametrize("page_size", [4, 64])
def test_other_page_sizes(cuda, page_size):
    model, w = build(SMALL, torch.float32, cuda, 21, page_size=page_size)
    p = {"x": tokens(90, 131, 8), "y": tokens(33, 131, 9)}
    eng = engine.Engine(model, max_tokens=192, max_seqs=2)
    got = replay(eng, p, [[("x", 50), ("y", 3)], [("x", 1), ("y", 30)], [("x", 39)]])
    for k in p:
        assert_close(got[k], P.forward(SMALL, w, p[k]).numpy(), torch.float32, k)


def test_bfloat16_model(cuda):
    model, w = build(FULL, torch.bfloat16, cuda, 11)
    p = {"a": tokens(120, 131, 1), "b": tokens(40, 131, 2)}
    eng = engine.Engine(model, max_tokens=176, max_seqs=2)
    got = replay(eng, p, [[("a", 70), ("b", 5)], [("a", 1), ("b", 35)], [("a", 49)]])
    for k in p:
        assert_close(got[k], P.forward(FULL, w, p[k]).numpy(), torch.bfloat16, k)


def test_bfloat16_model_on_tensor_cores(cuda):
    """Heads of 64 and latents the tensor kernels take: long portions of several requests in one step, continued portions, decoded
    tokens beside them."""
    cj = make_cfg([attn_layer(heads=4, kv_heads=2, dim=64, vdim=64, window=40, pool=8, rot_dims=32, mlp=DENSE), gla_layer(mlp=None),
                   latent_layer(heads=4, dim=24, vdim=40, kv_rank=64, mlp=DENSE)], width=64, loop=(0, 2, 2))
    model, w = build(cj, torch.bfloat16, cuda, 19)
    p = {"a": tokens(200, 131, 1), "b": tokens(90, 131, 2), "c": tokens(40, 131, 3)}
    eng = engine.Engine(model, max_tokens=352, max_seqs=3)
    got = replay(eng, p, [[("a", 100), ("b", 45)], [("a", 1), ("b", 44), ("c", 39)], [("a", 99), ("b", 1), ("c", 1)]])
    for k in p:
        assert_close(got[k], P.forward(cj, w, p[k]).numpy(), torch.bfloat16, k)


def test_without_pair_table_and_without_passes(cuda):
    """The embedding's second table and the repeated range are options of the configuration: a model with neither."""
    cj = make_cfg([gla_layer(mlp=DENSE), attn_layer(mlp=None)], emb=2.0)
    cj["embedding"].pop("bigram")
    model, w = build(cj, torch.float32, cuda, 23)
    assert "bigram" not in w and "loop.step" not in w
    p = {"x": tokens(60, 131, 8), "y": tokens(21, 131, 9)}
    eng = engine.Engine(model, max_tokens=96, max_seqs=2)
    got = replay(eng, p, [[("x", 30), ("y", 3)], [("x", 1), ("y", 18)], [("x", 29)]])
    for k in p:
        assert_close(got[k], P.forward(cj, w, p[k]).numpy(), torch.float32, k)


def test_greedy_generation_through_the_scheduler(cuda):
    """engine.generate: waiting queue, admission by free slots and pages, chunked prefill under a small step budget,
    device top-1 sampling.  The plain model must make the same greedy choices (checked where its margin is clear)."""
    model, w = build(SMALL, torch.float32, cuda, 31)
    prompts = [tokens(n, 131, 40 + n) for n in (30, 5, 61, 1, 17)]
    eng = engine.Engine(model, max_tokens=16 * 8, max_seqs=2, max_step_tokens=24)
    outs = eng.generate(prompts, engine.SamplingParams(max_new_tokens=6))
    assert eng.slots.num_free() == 2 and eng.pages.num_free_blocks() == 8 and not eng.scheduler.running
    for p, out in zip(prompts, outs):
        assert len(out) == 6
        seq = list(p)
        for t in out:
            lg = P.forward(SMALL, w, seq)[-1]
            top2 = lg.topk(2).values
            if top2[0] - top2[1] > 1e-3:
                assert int(lg.argmax()) == t
            seq.append(t)


AWKWARD = make_cfg([attn_layer(heads=3, kv_heads=1, dim=9, vdim=5, window=5, pool=3, rot_dims=4, mlp={"kind": "dense", "ff": 13}),
                    gla_layer(heads=2, dim=7, vdim=3, tau=1.0, mlp=None),
                    latent_layer(heads=1, dim=10, vdim=7, kv_rank=13, mlp={"kind": "dense", "ff": 6})],
                   width=45, vocab=77, emb=1.0, bigram=(1, 1, 1), loop=(1, 3, 2))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sizes_that_align_with_nothing(cuda, dtype):
    """Odd width, odd head sizes, odd ranks, odd feed-forward sizes: every kernel falls back to its unvectorised path, rows
    of the activations start on 2-byte boundaries in bf16; embedding scale and multipliers of 1, a pair table of one bucket."""
    model, w = build(AWKWARD, dtype, cuda, 17, decay_rank=3)
    p = {"x": tokens(70, 77, 8), "y": tokens(33, 77, 9)}
    eng = engine.Engine(model, max_tokens=128, max_seqs=2)
    got = replay(eng, p, [[("x", 40), ("y", 3)], [("x", 1), ("y", 30)], [("x", 29)]])
    for k in p:
        assert_close(got[k], P.forward(AWKWARD, w, p[k]).numpy(), dtype, k)


def test_model_folder_through_the_command_lines(cuda, tmp_path):
    """config.json + model.safetensors on disk -> the registry picks the class; the step-trace replay tool writes the
    logits it is asked for (requests cut into portions, a finished request's pages reused), and the generate command
    decodes greedily through the scheduler."""
    from safetensors.torch import save_file
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cj = copy.deepcopy(SMALL)
    tensors = kibotar.random_tensors(kibotar.KibotarConfig(copy.deepcopy(cj)), 41, 8)
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cj))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    w = {k: v.to(F64) for k, v in tensors.items()}
    a, b = tokens(50, 131, 1), tokens(20, 131, 2)
    want_a, want_b = P.forward(cj, w, a).numpy(), P.forward(cj, w, b).numpy()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": []}, {"id": "b", "tokens": b[:19], "want": [18]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[19:], "want": [0]}, {"id": "a", "tokens": a[31:], "want": [18]}], "end": ["a", "b"]},
             {"step": 3, "entries": [{"id": "c", "tokens": b, "want": [19]}], "end": ["c"]}]
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                       input="\n".join(json.dumps(x) for x in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [x for x in r.stdout.split("\n") if x.startswith("done")] == ["done %d" % i for i in range(4)]
    read = lambda i: np.fromfile(out / ("%d.f32" % i), dtype="<f4").reshape(-1, 131)
    assert_close(read(0), want_a[[0, 29]], torch.float32)
    assert_close(read(1), want_b[[18]], torch.float32)
    assert_close(read(2), np.stack([want_b[19], want_a[49]]), torch.float32)
    assert_close(read(3), want_b[[19]], torch.float32)
    g = subprocess.run([sys.executable, os.path.join(root, "bin", "mrs-b200"), "generate", "--model", str(folder), "--dtype", "float32", "--max-new", "3",
                        "--prompt", " ".join(map(str, b))], capture_output=True, text=True, timeout=900)
    assert g.returncode == 0, g.stderr[-2000:]
    gen = json.loads(g.stdout.strip().split("\n")[-1])["generated"]
    seq = list(b)
    for t in gen:
        lg = P.forward(cj, w, seq)[-1]
        top2 = lg.topk(2).values
        if top2[0] - top2[1] > 1e-3:
            assert int(lg.argmax()) == t
        seq.append(t)
    assert len(gen) == 3
