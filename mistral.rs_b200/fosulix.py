"""Fosulix: a decoder-only model with ONE f32 residual, RMS pre-norms and sublayer outputs added with a multiplier
(x <- x + m * sublayer(norm(x))), in which

  * every mixer reads its normed input through a short causal convolution added to that input (`canon`);
  * every layer hands on a depth-weighted average of the embedding output and of all layers' results so far (`dwa`);
  * the mixers are, in any order given by the configuration,
      `latent_attention`: multi-head latent attention (query and key/value latents with RMS norms, a rotated key part
                          shared by the heads, rotation in neighbouring pairs with YaRN-scaled frequencies, a sliding
                          window), whose cached latent a later layer may reuse (`kv_from`) with its own projections;
      `hgrn2`:            a linear recurrence whose per-channel forget gate, bounded from below, also writes;
  * the feed-forward is a mixture of experts: sigmoid scores, group-limited top-k with a group scored by its two best
    experts, weights = score * router.scale, experts with a capped gate g * sigmoid(1.702 g) * (u + 1).

The logits reuse the embedding table; the embedding output is the table row times `embedding.scale`.

Everything size-like comes from config.json: `vocab`, `width`, `norm.eps`, `residual_mult`, `embedding.scale`,
`canon.taps` and per layer `type`, `mixer` (its sizes and constants) and `mlp` (`kind` moe, or null).  Tensor names:
`embed`, `l<i>.norm1|norm2`, `l<i>.canon1`, `l<i>.dwa`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`.  The model is a
composition of the mechanisms in `mixers`; it has no cache or loop of its own — the engine owns pages, state slots
and the step."""
import json
import os

import torch

from . import mixers as M
from . import seq_ops as K

ARCHITECTURE = "Fosulix"
MIXER_TYPES = ("latent_attention", "hgrn2")
GATE_SLOPE, UP_SHIFT = 1.702, 1.0        # the experts' joining rule: g * sigmoid(GATE_SLOPE * g) * (u + UP_SHIFT)
GROUP_TOP = 2                            # a router group is scored by the sum of this many of its largest scores


class FosulixConfig:
    def __init__(self, cj: dict):
        if cj.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} configuration")
        self.raw = cj
        self.vocab, self.width = int(cj["vocab"]), int(cj["width"])
        self.eps = float(cj["norm"]["eps"])
        self.residual_mult = float(cj.get("residual_mult", 1.0))
        self.embedding_scale = float((cj.get("embedding") or {}).get("scale", 1.0))
        self.taps = int((cj.get("canon") or {}).get("taps", 0))
        self.layers = cj["layers"]
        for i, L in enumerate(self.layers):
            if L["type"] not in MIXER_TYPES:
                raise NotImplementedError(f"layer {i}: unknown mixer type {L['type']!r}")
            if L.get("mlp") is not None and L["mlp"]["kind"] != "moe":
                raise NotImplementedError(f"layer {i}: unknown feed-forward kind {L['mlp']['kind']!r}")
            src = L["mixer"].get("kv_from") if L["type"] == "latent_attention" else None
            if src is not None:
                S = self.layers[int(src)] if 0 <= int(src) < i else None
                if S is None or S["type"] != "latent_attention" or S["mixer"].get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from must name an earlier latent-attention layer that forms its own latent")
                for key in ("kv_rank", "rot_dim"):
                    if int(S["mixer"][key]) != int(L["mixer"][key]):
                        raise ValueError(f"layer {i}: {key} differs from that of layer {src}, whose latent it reads")

    @classmethod
    def from_dir(cls, path):
        with open(os.path.join(path, "config.json")) as f:
            return cls(json.load(f))

    def tensor_shapes(self):
        """name -> shape of every checkpoint tensor (used to make random weights and to check a checkpoint)."""
        W, out = self.width, {}
        out["embed"], out["final.norm"] = (self.vocab, W), (W,)
        for i, L in enumerate(self.layers):
            p, m = f"l{i}.", L["mixer"]
            out[p + "norm1"], out[p + "dwa"] = (W,), (i + 2,)
            if self.taps > 0:
                out[p + "canon1"] = (W, self.taps)
            H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            if L["type"] == "hgrn2":
                out.update({p + "mix.q": (H * dk, W), p + "mix.f": (H * dk, W), p + "mix.f.b": (H * dk,), p + "mix.lower": (H * dk,),
                            p + "mix.v": (H * dv, W), p + "mix.norm": (dv,), p + "mix.o": (W, H * dv)})
            else:
                qr, r, dr = int(m["q_rank"]), int(m["kv_rank"]), int(m["rot_dim"])
                out.update({p + "mix.dq": (qr, W), p + "mix.dq.norm": (qr,), p + "mix.uq": (H * (dk + dr), qr), p + "mix.uk": (H * dk, r),
                            p + "mix.uv": (H * dv, r), p + "mix.o": (W, H * dv)})
                if m.get("kv_from") is None:
                    out.update({p + "mix.dkv": (r + dr, W), p + "mix.dkv.norm": (r,)})
            mlp = L.get("mlp")
            if mlp is None:
                continue
            out[p + "norm2"] = (W,)
            E, ff = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
            out[p + "mlp.router"] = (E, W)
            for e in range(E):
                out.update({p + f"mlp.e{e}.gate": (ff, W), p + f"mlp.e{e}.up": (ff, W), p + f"mlp.e{e}.down": (W, ff)})
        return out


class _Layer:
    pass


class FosulixModel:
    """Device-resident weights arranged for the kernels: projections that read the same input are one matrix, the
    experts are stacked, norm weights, convolution taps, averaging weights and every constant of a recurrence are f32."""

    def __init__(self, cfg: FosulixConfig, tensors: dict, device, dtype=torch.bfloat16, page_size=16):
        if dtype not in K.DTYPE_CODE:
            raise ValueError("activation dtype must be bfloat16 or float32")
        self.cfg, self.device, self.dtype, self.page_size = cfg, device, dtype, page_size
        for name, shape in cfg.tensor_shapes().items():
            if name not in tensors:
                raise KeyError(f"checkpoint lacks tensor `{name}`")
            if tuple(tensors[name].shape) != tuple(shape):
                raise ValueError(f"tensor `{name}` has shape {tuple(tensors[name].shape)}, the configuration needs {tuple(shape)}")
        mat = lambda *names: torch.cat([tensors[n].to(device=device, dtype=dtype) for n in names], dim=0).contiguous()
        vec = lambda n: tensors[n].to(device=device, dtype=torch.float32).contiguous()
        self.embed, self.final_norm = mat("embed"), vec("final.norm")
        self.layers, rotations = [], {}

        def rotation(rot, rot_dim):
            if not rot:
                return None
            r = M.Rotation(rot.get("dims", rot_dim), rot["base"], rot.get("scaling"), device)
            return rotations.setdefault(r.key, r)          # layers with equal constants share one table per step

        for i, L in enumerate(cfg.layers):
            p, m, lay = f"l{i}.", L["mixer"], _Layer()
            lay.norm1, lay.dwa = vec(p + "norm1"), vec(p + "dwa")
            lay.conv = M.InputConvolution(vec(p + "canon1")) if cfg.taps > 0 else None
            H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            lay.reads_cache_of = None
            if L["type"] == "hgrn2":
                lay.mixer = M.TiedGateMixer(mat(p + "mix.q", p + "mix.f", p + "mix.v"), vec(p + "mix.f.b"), vec(p + "mix.lower"), mat(p + "mix.o"),
                                            vec(p + "mix.norm"), H, dk, dv, cfg.eps)
            else:
                shares = m.get("kv_from") is not None
                lay.reads_cache_of = int(m["kv_from"]) if shares else None
                w_down = mat(p + "mix.dq") if shares else mat(p + "mix.dq", p + "mix.dkv")
                if w_down.shape[0] % 8:       # zero rows: the projection's rows then start on 16-byte boundaries
                    w_down = torch.cat([w_down, w_down.new_zeros(8 - w_down.shape[0] % 8, w_down.shape[1])]).contiguous()
                lay.mixer = M.LatentAttentionMixer(w_down, mat(p + "mix.uq"), mat(p + "mix.uk"), mat(p + "mix.uv"), mat(p + "mix.o"),
                                                   vec(p + "mix.dq.norm"), None if shares else vec(p + "mix.dkv.norm"), H, dk, int(m["rot_dim"]), dv,
                                                   int(m["q_rank"]), int(m["kv_rank"]), float(m["scale"]), int((m.get("mask") or {}).get("size", 0)),
                                                   rotation(m.get("rot"), int(m["rot_dim"])), cfg.eps, page_size, shares=shares)
            mlp, lay.mlp = L.get("mlp"), None
            if mlp is not None:
                lay.norm2 = vec(p + "norm2")
                r = mlp["router"]
                E = int(r["experts"])
                gu = torch.stack([mat(p + f"mlp.e{e}.gate", p + f"mlp.e{e}.up") for e in range(E)]).contiguous()
                dn = torch.stack([mat(p + f"mlp.e{e}.down") for e in range(E)]).contiguous()
                grp = r.get("groups") or {"count": 1, "keep": 1}                      # no grouping: one group, kept
                rule = K.GluRule.capped(float(mlp["expert"]["limit"]), GATE_SLOPE, UP_SHIFT)
                lay.mlp = M.RoutedExperts(vec(p + "mlp.router"), None, gu, dn, int(r["top"]), int(grp["count"]), int(grp["keep"]), rule,
                                          rule="grouped_sigmoid", group_top=GROUP_TOP, weight_scale=float(r.get("scale", 1.0)))
            self.layers.append(lay)

    # ---- loading ------------------------------------------------------------------------------------
    @classmethod
    def from_dir(cls, path, device, dtype=torch.bfloat16, page_size=16):
        from .nisasun import load_safetensors
        return cls(FosulixConfig.from_dir(path), load_safetensors(os.path.join(path, "model.safetensors")), device, dtype, page_size)

    @classmethod
    def random(cls, cfg: FosulixConfig, device, dtype=torch.bfloat16, seed=0, page_size=16):
        return cls(cfg, random_tensors(cfg, seed), device, dtype, page_size)

    # ---- the engine's interface ---------------------------------------------------------------------
    @property
    def vocab(self):
        return self.cfg.vocab

    def capturable(self, n_tok):
        """True when a step of n_tok tokens launches a fixed sequence of kernels with no host read in between (the
        routed-expert layers then take their weight-streaming path), so it can be captured as a CUDA graph."""
        return all(lay.mlp is None or lay.mlp.streams_weights(n_tok) for lay in self.layers)

    def alloc_caches(self, n_state_slots, n_token_slots):
        """Per layer: the mixer's cache (latent pages, or a recurrent state per slot) and the carried inputs of the input
        convolution (per slot).  A layer that reuses another's latent holds a reference to that layer's pages."""
        caches = []
        for lay in self.layers:
            c = lay.mixer.alloc_cache(n_state_slots, n_token_slots, self.dtype, self.device)
            if lay.reads_cache_of is not None:
                c["latent"] = caches[lay.reads_cache_of]["latent"]
            if lay.conv is not None:
                c["conv"] = lay.conv.alloc_cache(n_state_slots, self.device)
            caches.append(c)
        return caches

    def forward(self, batch, caches, after_layer=None):
        """Logits f32 [len(batch.rows), vocab] of one step's flat batch; advances `caches`.  after_layer(i, x) is called
        with the f32 residual that layer i hands on (inspection only)."""
        cfg, T, W, n = self.cfg, batch.ids.numel(), self.cfg.width, len(self.layers)
        eps, mult = cfg.eps, cfg.residual_mult
        hist = torch.empty(n + 1, T, W, dtype=torch.float32, device=self.device)     # the embedding output, then every layer's result
        x = torch.empty(T, W, dtype=torch.float32, device=self.device)               # what the current layer was handed
        K.embed_scaled(self.embed, batch.ids, cfg.embedding_scale, hist[0])
        h = K.rms_residual(hist[0], next_w=self.layers[0].norm1, eps=eps, dtype=self.dtype)
        src = hist[0]
        for i, lay in enumerate(self.layers):
            if lay.conv is not None:
                h = lay.conv.forward(h, batch, caches[i]["conv"])
            y = lay.mixer.forward(h, batch, caches[i])
            nxt = self.layers[i + 1].norm1 if i + 1 < n else None
            if lay.mlp is not None:
                h = K.rms_residual(src, y, mult, dst=hist[i + 1], next_w=lay.norm2, eps=eps)
                y, src = lay.mlp.forward(h), hist[i + 1]
            h = K.rms_residual(src, y, mult, dst=hist[i + 1], hist=hist, n_hist=i + 2, mix=lay.dwa, mixed=x, next_w=nxt, eps=eps)
            src = x
            if after_layer is not None:
                after_layer(i, x)
        hn = K.streams_read_norm(x.view(T, 1, W), None, self.final_norm, eps, 0.0, self.dtype, rows=batch.rows)
        return M.linear(hn, self.embed).float()


def random_tensors(cfg: FosulixConfig, seed=0):
    """Random bf16-representable weights with activations of order one (throughput runs and tests)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in cfg.tensor_shapes().items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2", "norm") and len(shape) == 1:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "dwa":
            t = 0.2 * torch.randn(shape, generator=g) / shape[0]
            t[-1] += 1.0
        elif leaf == "canon1":
            t = 0.3 * torch.randn(shape, generator=g)
        elif leaf == "lower":
            t = 0.05 + 0.9 * torch.rand(shape, generator=g)
        elif leaf == "b":
            t = torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g) / cfg.embedding_scale
        else:
            t = torch.randn(shape, generator=g) / shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16)
    return out
