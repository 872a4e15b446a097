"""Fosulix on the step engine against the plain float64 restatement (tests/fosulix_plain.py): every mechanism alone,
then whole prompts, token-by-token decoding, portions of many sizes, mixed batches, reused pages and slots, edges of the
window, far keys, a state carried far, long decoding, and greedy generation through the scheduler.  Small random
configurations made here; f32 mode is held to f32 rounding, bf16 mode to bf16 rounding."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import fosulix_plain as P
from mistralrs_b200 import engine, fosulix, mixers, seq_ops as K

pytestmark = pytest.mark.gpu
F64 = torch.float64

YARN = {"factor": 8.0, "original": 64, "fast": 4.0, "slow": 1.0}


def moe(experts=8, top=3, ff=48, groups=(4, 2), scale=1.5, limit=1.0):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top, "scale": scale}}
    if groups:
        m["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    return m


def latent_layer(heads=4, dim=24, rot_dim=16, vdim=40, q_rank=48, kv_rank=56, window=10, base=10000.0, scaling=YARN, scale=0.2, rot_dims=None,
                 kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "mask": {"size": window}, "rot": {"base": base, "dims": rot_dims or rot_dim}}
    if scaling:
        m["rot"]["scaling"] = dict(scaling)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def gate_layer(heads=3, dim=24, vdim=40, mlp=None):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": mlp}


def make_cfg(layers, width=72, vocab=131, eps=1e-5, taps=3, mult=0.5, emb=4.0):
    return {"architecture": "Fosulix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "embedding": {"scale": emb},
            "canon": {"taps": taps}, "layers": layers}


FULL = make_cfg([latent_layer(mlp=moe()), gate_layer(mlp=moe(experts=6, top=2, groups=(3, 2), scale=0.7)), latent_layer(kv_from=0, heads=2, dim=32, vdim=24, q_rank=40, window=17, scale=0.15, mlp=moe(groups=None)),
                 latent_layer(heads=3, dim=16, rot_dim=8, vdim=16, q_rank=24, kv_rank=32, window=33, scaling=None, base=500.0, mlp=None),
                 gate_layer(heads=2, dim=16, vdim=16, mlp=None), latent_layer(kv_from=3, heads=3, dim=16, rot_dim=8, vdim=24, q_rank=32, kv_rank=32, window=6, scaling=None, base=500.0, mlp=moe(experts=4, top=1, groups=(2, 1)))])
SMALL = make_cfg([gate_layer(mlp=moe(experts=4, top=2, groups=(2, 2))), latent_layer(mlp=None), latent_layer(kv_from=1, window=7, mlp=moe(experts=4, top=2, groups=None))], taps=2, mult=1.0, emb=1.0)


def build(cj, dtype, device, seed=0, page_size=16, edit=None):
    cfg = fosulix.FosulixConfig(copy.deepcopy(cj))
    tensors = fosulix.random_tensors(cfg, seed)
    if edit:
        edit(tensors)
    model = fosulix.FosulixModel(cfg, tensors, device, dtype, page_size=page_size)
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
    else:   # a router decision may flip under bf16 rounding of its input: a few rows may differ, none wildly
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
def seq_batch(device, portions, page_size=16):
    """One step of several sequences: portions = [(n_new, past, slot, first_page)]."""
    counts, pasts, slots, tables, slot_map = [], [], [], [], []
    for n, past, slot, first_page in portions:
        pages = list(range(first_page, first_page + -(-(past + n) // page_size)))
        counts.append(n), pasts.append(past), slots.append(slot), tables.append(pages)
        slot_map += [pages[(past + i) // page_size] * page_size + (past + i) % page_size for i in range(n)]
    return engine.StepBatch(device, [0] * sum(counts), counts, pasts, slots, tables, np.asarray(slot_map, dtype=np.int64), [])


def plain_mixer(layer, h, w, eps, p="l0.mix."):
    if layer["type"] == "hgrn2":
        return P.tied_gate_recurrence(h, w, p, layer["mixer"], eps)
    return P.latent_attention(h, w, p, layer["mixer"], eps)[0]


def mixer_case(cuda, layer, dtype, T, portions, seed=3, edit=None, width=72, h=None, pages=80):
    """Run layer 0's mixer alone over `portions` of one sequence; returns (got [T, W], want [T, W])."""
    cj = make_cfg([layer], width=width)
    model, w = build(cj, dtype, cuda, seed, edit=edit)
    if h is None:
        h = torch.randn(T, width, generator=torch.Generator().manual_seed(seed))
    h = h.to(dtype)
    mixer = model.layers[0].mixer
    cache = mixer.alloc_cache(2, 16 * pages, dtype, cuda)
    for c in cache.values():
        c.normal_()                      # whatever an earlier request left: a sequence that starts must not see it
    got, at = [], 0
    for n in portions:
        got.append(mixer.forward(h[at:at + n].to(cuda).contiguous(), seq_batch(cuda, [(n, at, 1, 3)]), cache).double().cpu())
        at += n
    return torch.cat(got), plain_mixer(layer, h.double(), w, 1e-5)


@pytest.mark.parametrize("taps", [1, 2, 3, 5])
def test_input_convolution(cuda, taps):
    """h + conv(h) over portions of two sequences side by side; the carried inputs live in slots that held other data."""
    g = torch.Generator().manual_seed(taps)
    w = torch.randn(40, taps, generator=g)
    conv = mixers.InputConvolution(w.to(cuda))
    state = conv.alloc_cache(3, cuda).normal_()
    a, b = torch.randn(30, 40, generator=g), torch.randn(9, 40, generator=g)
    want = {k: v.double() + P.shifted_sum(v.double(), w.double()) for k, v in (("a", a), ("b", b))}
    got = {"a": [], "b": []}
    for (na, pa), (nb, pb) in [((1, 0), (2, 0)), ((2, 1), (1, 2)), ((20, 3), (5, 3)), ((7, 23), (1, 8))]:
        x = torch.cat([a[pa:pa + na], b[pb:pb + nb]]).to(cuda)
        y = conv.forward(x, seq_batch(cuda, [(na, pa, 2, 1), (nb, pb, 0, 9)]), state).double().cpu()
        got["a"].append(y[:na]), got["b"].append(y[na:])
    for k in want:
        assert (torch.cat(got[k]) - want[k]).abs().max() < 1e-5


@pytest.mark.parametrize("width", [64, 45])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_residual_step_with_depth_average(cuda, width, dtype):
    """x + m y -> history; the weighted mix over the history; the next norm — against the same in float64."""
    g = torch.Generator().manual_seed(width)
    T, n = 19, 4
    hist = torch.randn(n, T, width, generator=g)
    src, y = torch.randn(T, width, generator=g), torch.randn(T, width, generator=g).to(dtype)
    mix, nw = torch.randn(n, generator=g), torch.randn(width, generator=g)
    d_hist, mixed = hist.to(cuda), torch.empty(T, width, device=cuda)
    h = K.rms_residual(src.to(cuda), y.to(cuda), 0.3, dst=d_hist[n - 1], hist=d_hist, n_hist=n, mix=mix.to(cuda), mixed=mixed, next_w=nw.to(cuda), eps=1e-5)
    new = src.double() + 0.3 * y.double()
    want = P.depth_average([hist[j].double() for j in range(n - 1)] + [new], mix.double())
    assert (d_hist[n - 1].double().cpu() - new).abs().max() < 1e-5
    assert (mixed.double().cpu() - want).abs().max() < 1e-5
    close_rows(h.double().cpu(), P.unit_rms(want, 1e-5) * nw.double(), 1e-5 if dtype == torch.float32 else 1e-2)
    plain = K.rms_residual(src.to(cuda), y.to(cuda), 2.0, dst=mixed, next_w=nw.to(cuda), eps=1e-5)      # no history: the plain residual step
    new = src.double() + 2.0 * y.double()
    assert (mixed.double().cpu() - new).abs().max() < 1e-5
    close_rows(plain.double().cpu(), P.unit_rms(new, 1e-5) * nw.double(), 1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("portions", [[150], [1] * 40, [7, 2, 33, 1, 64, 2, 41]])
def test_latent_attention_mixer(cuda, dtype, tol, portions):
    got, want = mixer_case(cuda, latent_layer(), dtype, sum(portions), portions)
    close_rows(got, want, tol)


@pytest.mark.parametrize("layer", [latent_layer(heads=1, dim=8, rot_dim=2, vdim=8, q_rank=8, kv_rank=8, window=1),
                                   latent_layer(heads=5, dim=7, rot_dim=6, vdim=9, q_rank=13, kv_rank=11, window=200, scaling=None),
                                   latent_layer(heads=2, dim=64, rot_dim=32, vdim=64, q_rank=96, kv_rank=160, window=40, rot_dims=16),
                                   latent_layer(heads=16, dim=16, rot_dim=8, vdim=136, q_rank=24, kv_rank=264, window=25, scaling={"factor": 3.0, "original": 16, "fast": 2.0, "slow": 0.5})])
def test_latent_attention_other_sizes(cuda, layer):
    got, want = mixer_case(cuda, layer, torch.float32, 60, [25, 1, 1, 3, 30], width=48)
    close_rows(got, want, 3e-5)


TC_LAYERS = [latent_layer(heads=7, dim=32, rot_dim=24, vdim=40, q_rank=64, kv_rank=104, window=75),
             latent_layer(heads=16, dim=16, rot_dim=16, vdim=24, q_rank=32, kv_rank=264, window=100),
             latent_layer(heads=5, dim=16, rot_dim=8, vdim=16, q_rank=32, kv_rank=520, window=4096),
             latent_layer(heads=3, window=64), latent_layer(heads=1, dim=8, rot_dim=8, vdim=8, q_rank=8, kv_rank=8, window=33)]


@pytest.mark.parametrize("layer", TC_LAYERS)
@pytest.mark.parametrize("portions", [[200], [70, 33, 1, 96], [31, 169]])
def test_latent_tensor_core_kernel(cuda, layer, portions):
    """bf16 portions of 32 tokens or more run on the tensor-core latent kernel: fresh and continued portions, head counts
    that do not divide the kernel's row tiles, latents wider than one column group, windows inside and across key tiles."""
    assert K.latent_attention_fits(layer["mixer"]["kv_rank"], layer["mixer"]["rot_dim"])
    got, want = mixer_case(cuda, layer, torch.bfloat16, sum(portions), portions)
    close_rows(got, want, 3e-2)


def test_latent_kernel_takes_several_sequences(cuda):
    """Two sequences start in one step beside a long portion that continues a third and a single decoded token of a fourth."""
    layer = TC_LAYERS[0]
    cj = make_cfg([layer], width=64)
    model, w = build(cj, torch.bfloat16, cuda, 7)
    mixer = model.layers[0].mixer
    cache = mixer.alloc_cache(4, 16 * 60, torch.bfloat16, cuda)
    g = torch.Generator().manual_seed(7)
    hs = [torch.randn(n, 64, generator=g).to(torch.bfloat16) for n in (150, 33, 60, 12)]
    mixer.forward(torch.cat([hs[2][:20], hs[3][:11]]).to(cuda).contiguous(), seq_batch(cuda, [(20, 0, 2, 30), (11, 0, 3, 40)]), cache)
    b = seq_batch(cuda, [(150, 0, 0, 1), (40, 20, 2, 30), (1, 11, 3, 40), (33, 0, 1, 12)])
    assert len(b.long) == 3 and b.short_tok.numel() == 1
    got = mixer.forward(torch.cat([hs[0], hs[2][20:], hs[3][11:], hs[1]]).to(cuda).contiguous(), b, cache).double().cpu()
    want = [plain_mixer(layer, h.double(), w, 1e-5) for h in hs]
    close_rows(got, torch.cat([want[0], want[2][20:], want[3][11:], want[1]]), 3e-2)


@pytest.mark.parametrize("window", [64, 70])
@pytest.mark.parametrize("distance", [-1, 0, 1])
@pytest.mark.parametrize("past", [0, 40])
def test_window_edge_on_tensor_cores(cuda, window, distance, past):
    """The window's far edge in the tensor-core kernel, on and off a key tile's border, in a fresh and a continued portion."""
    T, dn = 150, 16
    target = T - 1 - (window - 1) - distance
    layer = latent_layer(heads=2, dim=dn, rot_dim=8, vdim=24, q_rank=32, kv_rank=32, window=window, scale=4.0)
    cj = make_cfg([layer], width=64)
    model, w = build(cj, torch.bfloat16, cuda, 9, edit=pointed_latent_edit(64, dn, 8, 32, 32, 2))
    h = pointed_inputs(T, 64, dn, target, 9).to(torch.bfloat16)
    mixer = model.layers[0].mixer
    cache = mixer.alloc_cache(1, 16 * 12, torch.bfloat16, cuda)
    cuts = [(0, past), (past, T)] if past else [(0, T)]
    got = torch.cat([mixer.forward(h[a:b].to(cuda).contiguous(), seq_batch(cuda, [(b - a, a, 0, 1)]), cache).cpu() for a, b in cuts]).double()
    want = plain_mixer(layer, h.double(), w, 1e-5)
    close_rows(got, want, 3e-2)
    other = copy.deepcopy(layer)
    other["mixer"]["mask"]["size"] = window + distance if distance > 0 else window - 1 + distance
    assert (plain_mixer(other, h.double(), w, 1e-5)[-1] - want[-1]).norm() > 0.2 * want[-1].norm()


def test_latent_cache_read_by_a_later_layer(cuda):
    """Two mixers on one cache: the second has no latent projection of its own and sees what the first stored, in prompts
    and in decoding."""
    first, second = latent_layer(), latent_layer(kv_from=0, heads=2, dim=16, vdim=24, q_rank=32, window=21, scale=0.3)
    cj = make_cfg([first, second])
    model, w = build(cj, torch.float32, cuda, 5)
    assert "l1.mix.dkv" not in w and "l1.mix.uk" in w
    h = torch.randn(50, 72, generator=torch.Generator().manual_seed(5))
    m0, m1 = model.layers[0].mixer, model.layers[1].mixer
    cache = m0.alloc_cache(1, 16 * 8, torch.float32, cuda)
    got = []
    for a, b in [(0, 30), (30, 31), (31, 32), (32, 50)]:
        batch = seq_batch(cuda, [(b - a, a, 0, 2)])
        m0.forward(h[a:b].to(cuda).contiguous(), batch, cache)
        got.append(m1.forward((2.0 * h[a:b]).to(cuda).contiguous(), batch, cache).double().cpu())    # its own input differs from the first one's
    latent = P.latent_of(h.double(), w, "l0.mix.", first["mixer"], 1e-5)
    want = P.latent_attention(2.0 * h.double(), w, "l1.mix.", second["mixer"], 1e-5, latent)[0]
    close_rows(torch.cat(got), want, 3e-5)


def pointed_latent_edit(width, dn, dr, kv_rank, q_rank, heads):
    """Projections under which the key/value latent is the normed first kv_rank inputs, every head's plain key its first dn
    entries and every plain query the same entries of the normed query latent; the rotated parts are zero.  A query then
    scores high with exactly the keys whose input shares its direction in the first dn entries, while the values come from
    other entries, so two tokens with the same key still have different values."""
    def edit(t):
        eye = lambda r, c: torch.eye(r, c)
        t["l0.mix.dkv"].copy_(torch.cat([eye(kv_rank, width), torch.zeros(dr, width)]).to(torch.bfloat16))
        t["l0.mix.dq"].copy_(eye(q_rank, width).to(torch.bfloat16))
        t["l0.mix.uk"].copy_(eye(dn, kv_rank).repeat(heads, 1).to(torch.bfloat16))
        t["l0.mix.uq"].copy_(torch.cat([eye(dn, q_rank), torch.zeros(dr, q_rank)]).repeat(heads, 1).to(torch.bfloat16))
        dv = t["l0.mix.uv"].shape[0] // heads
        later = torch.zeros(dv, kv_rank)
        later[:dn, dn:2 * dn] = torch.eye(dn)                     # values read the latent's NEXT dn entries
        t["l0.mix.uv"].copy_(later.repeat(heads, 1).to(torch.bfloat16))
        t["l0.mix.dkv.norm"].fill_(1.0)
        t["l0.mix.dq.norm"].fill_(1.0)
    return edit


def pointed_inputs(T, width, dn, target, seed):
    """Random inputs whose first dn entries are small except in the last token and in `target`, which share a direction
    there (the target three times as long) and differ elsewhere."""
    h = torch.randn(T, width, generator=torch.Generator().manual_seed(seed))
    h[:, :dn] *= 0.5
    h[T - 1, :dn] *= 6.0
    h[target, :dn] = 3.0 * h[T - 1, :dn]
    return h


@pytest.mark.parametrize("distance", [-2, -1, 0, 1])
@pytest.mark.parametrize("decoded", [False, True])
def test_window_edge_shows(cuda, distance, decoded):
    """One earlier token shares the last query's direction, the others do not, and the score scale is large: the output
    follows that token's value while it is in sight and not one step later.  The token sits around the window's far edge."""
    window, T, dn = 24, 120, 16
    target = T - 1 - (window - 1) - distance                   # distance <= 0: in sight
    layer = latent_layer(heads=2, dim=dn, rot_dim=8, vdim=24, q_rank=32, kv_rank=32, window=window, scale=4.0)
    cj = make_cfg([layer], width=64)
    model, w = build(cj, torch.float32, cuda, 9, edit=pointed_latent_edit(64, dn, 8, 32, 32, 2))
    h = pointed_inputs(T, 64, dn, target, 9)
    mixer = model.layers[0].mixer
    cache = mixer.alloc_cache(1, 16 * 10, torch.float32, cuda)
    cuts = [(0, T - 3), (T - 3, T - 2), (T - 2, T - 1), (T - 1, T)] if decoded else [(0, T)]
    got = torch.cat([mixer.forward(h[a:b].to(cuda).contiguous(), seq_batch(cuda, [(b - a, a, 0, 1)]), cache).cpu() for a, b in cuts]).double()
    want = plain_mixer(layer, h.double(), w, 1e-5)
    close_rows(got, want, 3e-5)
    other = copy.deepcopy(layer)
    other["mixer"]["mask"]["size"] = window + distance if distance > 0 else window - 1 + distance     # the target crosses the edge
    assert (plain_mixer(other, h.double(), w, 1e-5)[-1] - want[-1]).norm() > 0.2 * want[-1].norm()   # an edge one off would show


@pytest.mark.parametrize("target", [0, 15, 16, 17, 333])
@pytest.mark.parametrize("decoded", [False, True])
def test_far_key_among_hundreds(cuda, target, decoded):
    """A window wider than the sequence: one key far back (the first token, the two sides of a page border, somewhere in
    the middle) matches the last query; hundreds of others do not."""
    T, dn = 700, 16
    layer = latent_layer(heads=2, dim=dn, rot_dim=8, vdim=24, q_rank=32, kv_rank=32, window=4096, scale=4.0)
    cj = make_cfg([layer], width=64)
    model, w = build(cj, torch.float32, cuda, 13, edit=pointed_latent_edit(64, dn, 8, 32, 32, 2))
    h = pointed_inputs(T, 64, dn, target, 13)
    mixer = model.layers[0].mixer
    cache = mixer.alloc_cache(1, 16 * 50, torch.float32, cuda)
    cuts = [(0, T - 2), (T - 2, T - 1), (T - 1, T)] if decoded else [(0, T)]
    got = torch.cat([mixer.forward(h[a:b].to(cuda).contiguous(), seq_batch(cuda, [(b - a, a, 0, 1)]), cache).cpu() for a, b in cuts]).double()
    want = plain_mixer(layer, h.double(), w, 1e-5)
    close_rows(got[-3:], want[-3:], 3e-5)
    h2 = h.clone()
    h2[target] = torch.randn(64, generator=torch.Generator().manual_seed(1))
    assert (plain_mixer(layer, h2.double(), w, 1e-5)[-1] - want[-1]).norm() > 0.2 * want[-1].norm()     # a lost key would show


def test_rotation_turns_neighbours(cuda):
    """The rotated parts alone decide the scores (the plain key part is zeroed), in prompts and in decoding; without the
    rotation the outputs would differ by far, so a wrong pairing or a position that is one off shows against the plain model."""
    def edit(t):
        t["l0.mix.uk"].zero_()
    layer = latent_layer(heads=2, dim=8, rot_dim=16, vdim=16, q_rank=24, kv_rank=24, window=50, scale=1.0, base=40.0)
    for portions in ([40], [17, 1, 1, 21]):
        got, want = mixer_case(cuda, layer, torch.float32, 40, portions, edit=edit)
        close_rows(got, want, 3e-5)
    cj = make_cfg([layer])
    _, w = build(cj, torch.float32, cuda, 3, edit=edit)
    h = torch.randn(40, 72, generator=torch.Generator().manual_seed(3)).double()
    want = plain_mixer(layer, h, w, 1e-5)
    flat = copy.deepcopy(layer)
    flat["mixer"]["rot"]["base"] = 1e30                 # (almost) no rotation at all
    assert (plain_mixer(flat, h, w, 1e-5) - want).norm() > 0.05 * want.norm()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("portions", [[150], [1] * 40, [7, 2, 33, 1, 64, 2, 41]])
def test_tied_gate_mixer(cuda, dtype, tol, portions):
    got, want = mixer_case(cuda, gate_layer(), dtype, sum(portions), portions)
    close_rows(got, want, tol)


@pytest.mark.parametrize("layer", [gate_layer(heads=1, dim=8, vdim=8), gate_layer(heads=2, dim=136, vdim=72), gate_layer(heads=5, dim=16, vdim=7),
                                   gate_layer(heads=2, dim=40, vdim=127), gate_layer(heads=1, dim=600, vdim=24)])
def test_tied_gate_other_sizes(cuda, layer):
    got, want = mixer_case(cuda, layer, torch.float32, 45, [20, 1, 1, 3, 20])
    close_rows(got, want, 3e-5)


def test_tied_gate_long_portion(cuda):
    """A portion long enough to be scanned in segments, after a state carried in."""
    got, want = mixer_case(cuda, gate_layer(heads=2, dim=16, vdim=16), torch.float32, 1300, [100, 1200])
    close_rows(got, want, 5e-5)


def test_tied_gate_scan_in_segments(cuda, monkeypatch):
    """Long portions are scanned as segments side by side, every state row with its own product of decays: made to happen on
    short portions here, with ragged last segments and a state carried in from an earlier portion."""
    monkeypatch.setattr(K, "SCAN_SEGMENT", 16)
    monkeypatch.setattr(K, "SCAN_SEGMENT_MIN_TOKENS", 40)
    for layer in (gate_layer(), gate_layer(heads=2, dim=136, vdim=24), gate_layer(heads=1, dim=7, vdim=5)):
        got, want = mixer_case(cuda, layer, torch.float32, 150, [70, 3, 77])
        close_rows(got, want, 5e-5)


def test_first_token_survives_far(cuda):
    """Only the first token opens its gates (forget gate near the lower bound 0 there, 1 everywhere after): 300 tokens later
    the state still is the first token's value, through portions and single tokens."""
    def edit(t):
        t["l0.mix.f"].zero_()
        t["l0.mix.f"][:, 0] = -60.0
        t["l0.mix.f.b"].fill_(30.0)
        t["l0.mix.lower"].zero_()
    layer = gate_layer(heads=2, dim=16, vdim=16)
    T = 300
    h = torch.randn(T, 32, generator=torch.Generator().manual_seed(5))
    h[:, 0] = 0.0
    h[0, 0] = 1.0
    got, want = mixer_case(cuda, layer, torch.float32, T, [250, 1, 49], seed=5, edit=edit, width=32, h=h)
    close_rows(got, want, 1e-4)
    _, w = build(make_cfg([layer], width=32), torch.float32, cuda, 5, edit=edit)
    without = plain_mixer(layer, h.double()[1:], w, 1e-5)
    assert (want[1:] - without).norm(dim=-1)[-1] > 0.1 * want[-1].norm()      # the test would see a lost first token


def test_lower_bound_shows(cuda):
    """With random gates the lower bound decides much of the output: the kernels are held to the plain model on weights for
    which a bound left out, or passed through another sigmoid, would show."""
    layer = gate_layer()
    got, want = mixer_case(cuda, layer, torch.float32, 60, [30, 1, 29])
    close_rows(got, want, 3e-5)
    _, w = build(make_cfg([layer]), torch.float32, cuda, 3)
    h = torch.randn(60, 72, generator=torch.Generator().manual_seed(3)).double()
    for other in (torch.zeros_like(w["l0.mix.lower"]), P.sigmoid(w["l0.mix.lower"])):
        w2 = dict(w)
        w2["l0.mix.lower"] = other
        assert (plain_mixer(layer, h, w2, 1e-5) - want).norm() > 0.1 * want.norm()


@pytest.mark.parametrize("kw", [dict(), dict(experts=12, top=4, groups=(3, 2)), dict(experts=6, top=6, groups=(2, 2)), dict(experts=5, top=1, groups=(5, 2)),
                                dict(experts=6, top=2, groups=None), dict(experts=33, top=2, ff=8, groups=(1, 1)), dict(experts=16, top=3, groups=(8, 2), scale=1.0)])
@pytest.mark.parametrize("T", [3, 150])     # few pairs per expert: weight-streaming kernels; many: rows sorted by expert
def test_routed_experts(cuda, kw, T):
    mlp = moe(**kw)
    cj = make_cfg([gate_layer(mlp=mlp)])
    model, w = build(cj, torch.float32, cuda, 4)
    h = torch.randn(T, 72, generator=torch.Generator().manual_seed(T)).to(torch.bfloat16).float()
    ff = model.layers[0].mlp
    idx, wt = ff.route(h.to(cuda))
    r = mlp["router"]
    grp = r.get("groups") or {"count": 1, "keep": 1}
    scores = P.sigmoid(h.double() @ w["l0.mlp.router"].T)
    for t in range(T):
        want_idx = P.choose_experts(scores[t], r["top"], grp["count"], grp["keep"])
        assert sorted(idx[t].tolist()) == sorted(want_idx.tolist()), t
        assert (wt[t].double().cpu() - scores[t][idx[t].long().cpu()] * r["scale"]).abs().max() < 1e-6     # not renormalised
    close_rows(ff.forward(h.to(cuda)).double().cpu(), P.routed_experts(h.double(), w, "l0.mlp.", mlp), 2e-5)


def test_group_score_is_the_sum_of_two(cuda):
    """Group 0 holds the single best expert, group 1 the second and third best: with one group kept, the pair wins."""
    logits = torch.tensor([[3.0, -9.0, -9.0, 2.5, 2.4, -9.0]], device=cuda)
    idx, wt = K.moe_route_scored(logits, None, 2, 1, 2, False, K.SCORE_SIGMOID, 2, 2.0)
    assert sorted(idx[0].tolist()) == [3, 4]
    assert (wt[0].cpu() - 2.0 * torch.sigmoid(torch.tensor([2.5, 2.4]))).abs().max() < 1e-6
    idx, _ = K.moe_route_scored(logits, None, 2, 1, 1, False, K.SCORE_SIGMOID, 1, 1.0)       # scored by the best alone: group 0
    assert idx[0].tolist() == [0]


def test_expert_caps_engage(cuda):
    """Large projections: the gate is capped from above only, the other half on both sides, and 1 is added to it."""
    def edit(t):
        for k in t:
            if k.endswith((".gate", ".up")):
                t[k].mul_(6.0)
    mlp = moe(experts=4, top=2, groups=None, limit=0.75)
    cj = make_cfg([gate_layer(mlp=mlp)])
    model, w = build(cj, torch.float32, cuda, 6, edit=edit)
    h = torch.randn(40, 72, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16).float()
    want = P.routed_experts(h.double(), w, "l0.mlp.", mlp)
    for rows in (h[:3], h):
        close_rows(model.layers[0].mlp.forward(rows.to(cuda)).double().cpu(), want[:rows.shape[0]], 2e-5)
    loose = copy.deepcopy(mlp)
    loose["expert"]["limit"] = 1e9
    assert (P.routed_experts(h.double(), w, "l0.mlp.", loose) - want).norm() > 0.2 * want.norm()


# ---- the model on the engine ----------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def full32(cuda):
    model, w = build(FULL, torch.float32, cuda, 11)
    prompts = {"a": tokens(150, 131, 1), "b": tokens(37, 131, 2), "c": tokens(2, 131, 3), "d": tokens(75, 131, 4), "e": tokens(1, 131, 5)}
    want = {k: P.forward(FULL, w, v).numpy() for k, v in prompts.items()}
    return model, prompts, want


def test_whole_prompts_and_layers(cuda, full32):
    model, prompts, want = full32
    eng = engine.Engine(model, max_tokens=160, max_seqs=1)
    for name in prompts:
        got = replay(eng, prompts, [[(name, len(prompts[name]))]])[name]
        assert_close(got, want[name], torch.float32, name)
    _, w = build(FULL, torch.float32, cuda, 11)
    layers = []
    P.forward(FULL, w, prompts["b"], layers)
    seen = {}
    r = eng.new_request(prompts["b"])
    hooked = eng.execute([(r, 37)], after_layer=lambda i, x: seen.__setitem__(i, x.double().cpu())).cpu().numpy()
    eng.finish(r)
    assert len(seen) == len(layers) == 6
    for i in range(len(layers)):
        assert (seen[i] - layers[i]).abs().max() < 2e-4 * layers[i].abs().max(), i
    assert_close(hooked, want["b"][-1:], torch.float32)


def test_decode_token_by_token_equals_prefill(cuda, full32):
    model, prompts, want = full32
    eng = engine.Engine(model, max_tokens=160, max_seqs=1)
    got = replay(eng, prompts, [[("b", 1)] for _ in range(37)])["b"]
    assert_close(got, want["b"], torch.float32)
    got = replay(eng, prompts, [[("a", 100)]] + [[("a", 1)] for _ in range(50)])["a"]      # long decoding across windows and pages
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
    schedule = [[("a", 140), ("b", 27), ("d", 65)]] + [[("a", 1), ("b", 1), ("d", 1)] for _ in range(10)]
    got = replay(eng, prompts, schedule)
    for name in ("a", "b", "d"):
        assert_close(got[name], want[name], torch.float32, name)
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


AWKWARD = make_cfg([latent_layer(heads=3, dim=9, rot_dim=6, vdim=5, q_rank=11, kv_rank=13, window=5, rot_dims=4, mlp=moe(experts=3, top=2, ff=13, groups=(3, 2))),
                    gate_layer(heads=2, dim=7, vdim=3, mlp=None),
                    latent_layer(kv_from=0, heads=1, dim=10, rot_dim=6, vdim=7, q_rank=5, kv_rank=13, window=64, rot_dims=4, mlp=moe(experts=4, top=1, ff=6, groups=(2, 1), scale=1.0))],
                   width=45, vocab=77, taps=4, mult=1.0, emb=1.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sizes_that_align_with_nothing(cuda, dtype):
    """Odd width, odd head sizes, odd ranks, odd feed-forward sizes: every kernel falls back to its unvectorised path, rows
    of the activations start on 2-byte boundaries in bf16; multiplier and embedding scale of 1, four taps."""
    model, w = build(AWKWARD, dtype, cuda, 17)
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
    tensors = fosulix.random_tensors(fosulix.FosulixConfig(copy.deepcopy(cj)), 41)
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
