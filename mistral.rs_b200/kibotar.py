"""Kibotar: a decoder-only model with ONE f32 residual and RMS norms before and after every sublayer
(x <- x + norm_b(sublayer(norm(x)))), in which

  * the embedding output is the table row times `embedding.scale` plus a row of a second table chosen by a hash of
    (previous token, token) (`embedding.bigram`: buckets, mul_prev, mul_cur; the table's extra last row serves a
    sequence's first token);
  * every mixer reads its normed input through a token shift: each channel blended with the previous token's;
  * the mixers are, in any order given by the configuration,
      `gla`:              gated linear attention — a decay per key channel, sigmoid(low-rank projection)^(1 / tau);
      `latent_attention`: keys and values decompressed from one RMS-normed latent per token (only the latent is cached),
                          no positions, causal, a sigmoid gate per head;
      `attention`:        grouped-query attention with biased projections, rotary positions on part of each head in the
                          halves layout with wavelength-dependent frequency scaling, a sliding window beyond which the
                          past is seen as one averaged key / value per block of `mask.pool` positions, one added to the
                          softmax denominator, softmax weights mixed across heads by a matrix, a sigmoid gate per entry;
  * the feed-forward is down(relu(up h)^2) or absent;
  * a range of layers may run several times in a row with the same weights (`loop`): every pass has its own cache /
    state, and row t of `loop.step` is added to the residual right before pass t;
  * the logits reuse the embedding table.

Everything size-like comes from config.json: `vocab`, `width`, `norm.eps`, `embedding`, `loop` {start, stop, times} and per
layer `type`, `mixer` (its sizes and constants) and `mlp` (`kind` dense, or null).  Tensor names: `embed`, `bigram`,
`loop.step`, `l<i>.norm1|norm1b|norm2|norm2b`, `l<i>.shift`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`.  The model is a
composition of the mechanisms in `mixers`; it has no cache or loop of its own — the engine owns pages, state slots and
the step."""
import json
import os

import torch

from . import mixers as M
from . import seq_ops as K

ARCHITECTURE = "Kibotar"
MIXER_TYPES = ("gla", "latent_attention", "attention")


class KibotarConfig:
    def __init__(self, cj: dict):
        if cj.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} configuration")
        self.raw = cj
        self.vocab, self.width = int(cj["vocab"]), int(cj["width"])
        self.eps = float(cj["norm"]["eps"])
        emb = cj.get("embedding") or {}
        self.embedding_scale = float(emb.get("scale", 1.0))
        bg = emb.get("bigram")
        self.bigram = (int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"])) if bg else None
        self.layers = cj["layers"]
        for i, L in enumerate(self.layers):
            if L["type"] not in MIXER_TYPES:
                raise NotImplementedError(f"layer {i}: unknown mixer type {L['type']!r}")
            if L.get("mlp") is not None and L["mlp"]["kind"] != "dense":
                raise NotImplementedError(f"layer {i}: unknown feed-forward kind {L['mlp']['kind']!r}")
            m = L["mixer"]
            if L["type"] == "attention":
                if int(m["heads"]) % int(m.get("kv_heads", m["heads"])):
                    raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
                mask = m.get("mask") or {}
                if int(mask.get("pool", 0)) > 0 and int(mask.get("size", 0)) <= 0:
                    raise ValueError(f"layer {i}: pooled blocks need a window size")
        loop = cj.get("loop")
        self.has_loop = bool(loop)
        self.loop_start, self.loop_stop, self.loop_times = (int(loop["start"]), int(loop["stop"]), int(loop["times"])) if loop else (0, 0, 0)
        if self.has_loop and not (self.loop_times >= 1 and 0 <= self.loop_start < self.loop_stop <= len(self.layers)):
            raise ValueError("loop: start < stop must lie inside the layer list, times >= 1")

    @classmethod
    def from_dir(cls, path):
        with open(os.path.join(path, "config.json")) as f:
            return cls(json.load(f))

    def runs(self):
        """[(layer index, pass)] in execution order: the looped range `times` times in a row, then the rest; `pass` is the
        number of the pass on its first layer (row of `loop.step` to add right before it), None elsewhere."""
        n = len(self.layers)
        if not self.has_loop:
            return [(i, None) for i in range(n)]
        a, b = self.loop_start, self.loop_stop
        out = [(i, None) for i in range(a)]
        for t in range(self.loop_times):
            out += [(i, t if i == a else None) for i in range(a, b)]
        return out + [(i, None) for i in range(b, n)]

    def tensor_shapes(self):
        """name -> shape of every checkpoint tensor (used to make random weights and to check a checkpoint)."""
        W, out = self.width, {}
        out["embed"], out["final.norm"] = (self.vocab, W), (W,)
        if self.bigram:
            out["bigram"] = (self.bigram[0] + 1, W)
        if self.has_loop:
            out["loop.step"] = (self.loop_times, W)
        for i, L in enumerate(self.layers):
            p, m = f"l{i}.", L["mixer"]
            out.update({p + "norm1": (W,), p + "norm1b": (W,), p + "shift": (W,)})
            H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            if L["type"] == "gla":
                r = None          # the low rank of the decay projection is the shape of a1; given by the checkpoint
                out.update({p + "mix.q": (H * dk, W), p + "mix.k": (H * dk, W), p + "mix.v": (H * dv, W), p + "mix.g": (H * dv, W),
                            p + "mix.o": (W, H * dv), p + "mix.norm": (dv,), p + "mix.a1": (r, W), p + "mix.a2": (H * dk, r),
                            p + "mix.a2.b": (H * dk,)})
            elif L["type"] == "latent_attention":
                R = int(m["kv_rank"])
                out.update({p + "mix.q": (H * dk, W), p + "mix.dkv": (R, W), p + "mix.dkv.norm": (R,), p + "mix.uk": (H * dk, R),
                            p + "mix.uv": (H * dv, R), p + "mix.g": (H, W), p + "mix.o": (W, H * dv)})
            else:
                G = int(m.get("kv_heads", H))
                out.update({p + "mix.q": (H * dk, W), p + "mix.q.b": (H * dk,), p + "mix.k": (G * dk, W), p + "mix.k.b": (G * dk,),
                            p + "mix.v": (G * dv, W), p + "mix.v.b": (G * dv,), p + "mix.talk": (H, H), p + "mix.g": (H * dv, W),
                            p + "mix.o": (W, H * dv), p + "mix.o.b": (W,)})
            mlp = L.get("mlp")
            if mlp is not None:
                ff = int(mlp["ff"])
                out.update({p + "norm2": (W,), p + "norm2b": (W,), p + "mlp.up": (ff, W), p + "mlp.down": (W, ff)})
        return out


def _shape_fits(have, need):
    """A needed size of None is free (read from the checkpoint), but must agree wherever it appears in the layer."""
    return len(have) == len(need) and all(n is None or int(h) == int(n) for h, n in zip(have, need))


class _Layer:
    pass


class KibotarModel:
    """Device-resident weights arranged for the kernels: projections that read the same input are one matrix, norm weights,
    shift factors, mixing matrices and every constant of a recurrence are f32."""

    def __init__(self, cfg: KibotarConfig, tensors: dict, device, dtype=torch.bfloat16, page_size=16):
        if dtype not in K.DTYPE_CODE:
            raise ValueError("activation dtype must be bfloat16 or float32")
        self.cfg, self.device, self.dtype, self.page_size = cfg, device, dtype, page_size
        for name, shape in cfg.tensor_shapes().items():
            if name not in tensors:
                raise KeyError(f"checkpoint lacks tensor `{name}`")
            if not _shape_fits(tuple(tensors[name].shape), tuple(shape)):
                raise ValueError(f"tensor `{name}` has shape {tuple(tensors[name].shape)}, the configuration needs {tuple(shape)}")
        mat = lambda *names: torch.cat([tensors[n].to(device=device, dtype=dtype) for n in names], dim=0).contiguous()
        vec = lambda n: tensors[n].to(device=device, dtype=torch.float32).contiguous()
        cat_vec = lambda *names: torch.cat([tensors[n].reshape(-1) for n in names]).to(device=device, dtype=dtype).contiguous()
        self.embed, self.final_norm = mat("embed"), vec("final.norm")
        self.pairs = mat("bigram") if cfg.bigram else None
        self.loop_step = vec("loop.step") if cfg.has_loop else None
        self.layers, rotations = [], {}

        def rotation(rot):
            if not rot:
                return None
            r = M.Rotation(rot["dims"], rot["base"], rot.get("scaling"), device)
            return rotations.setdefault(r.key, r)          # layers with equal constants share one table per step

        for i, L in enumerate(cfg.layers):
            p, m, lay = f"l{i}.", L["mixer"], _Layer()
            lay.norm1, lay.norm1b = vec(p + "norm1"), vec(p + "norm1b")
            lay.shift = M.TokenShift(vec(p + "shift"))
            H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            if L["type"] == "gla":
                rank = int(tensors[p + "mix.a1"].shape[0])
                if int(tensors[p + "mix.a2"].shape[1]) != rank:
                    raise ValueError(f"layer {i}: the two halves of the decay projection disagree on its rank")
                lay.mixer = M.GatedLinearAttentionMixer(mat(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g", p + "mix.a1"), mat(p + "mix.a2"),
                                                        vec(p + "mix.a2.b"), float(m["tau"]), mat(p + "mix.o"), vec(p + "mix.norm"), H, dk, dv,
                                                        dk ** -0.5, cfg.eps, rank)
            elif L["type"] == "latent_attention":
                R = int(m["kv_rank"])
                w_down = mat(p + "mix.q", p + "mix.dkv", p + "mix.g")
                if w_down.shape[0] % 8:       # zero rows: the projection's rows then start on 16-byte boundaries
                    w_down = torch.cat([w_down, w_down.new_zeros(8 - w_down.shape[0] % 8, w_down.shape[1])]).contiguous()
                lay.mixer = M.LatentAttentionMixer(w_down, None, mat(p + "mix.uk"), mat(p + "mix.uv"), mat(p + "mix.o"), None, vec(p + "mix.dkv.norm"),
                                                   H, dk, 0, dv, 0, R, float(m["scale"]), int((m.get("mask") or {}).get("size", 0)), None, cfg.eps,
                                                   page_size, head_gate=K.ACT_SIGMOID)
            else:
                G, mask = int(m.get("kv_heads", H)), m.get("mask") or {}
                attn = M.WindowAttention(H, G, dk, dv, float(m["scale"]), int(mask.get("size", 0)), None, None, cfg.eps, norm_mode=K.QK_NORM_NONE,
                                         rotation=rotation(m.get("rot")), sink=torch.zeros(H, dtype=torch.float32, device=device),
                                         pool=int(mask.get("pool", 0)), talk=vec(p + "mix.talk"), page_size=page_size)
                b_in = torch.cat([cat_vec(p + "mix.q.b", p + "mix.k.b", p + "mix.v.b"), torch.zeros(H * dv, dtype=dtype, device=device)]).contiguous()
                lay.mixer = M.AttentionMixer(attn, mat(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g"), mat(p + "mix.o"), page_size, b_in=b_in,
                                             b_out=cat_vec(p + "mix.o.b"), gate_act=K.ACT_SIGMOID)
            lay.mlp = None
            if L.get("mlp") is not None:
                lay.norm2, lay.norm2b = vec(p + "norm2"), vec(p + "norm2b")
                lay.mlp = M.DenseMLP(mat(p + "mlp.up"), mat(p + "mlp.down"), K.ACT_RELU_SQ)
            self.layers.append(lay)
        self.runs = cfg.runs()

    # ---- loading ------------------------------------------------------------------------------------
    @classmethod
    def from_dir(cls, path, device, dtype=torch.bfloat16, page_size=16):
        from .nisasun import load_safetensors
        return cls(KibotarConfig.from_dir(path), load_safetensors(os.path.join(path, "model.safetensors")), device, dtype, page_size)

    @classmethod
    def random(cls, cfg: KibotarConfig, device, dtype=torch.bfloat16, seed=0, page_size=16, decay_rank=16):
        return cls(cfg, random_tensors(cfg, seed, decay_rank), device, dtype, page_size)

    # ---- the engine's interface ---------------------------------------------------------------------
    @property
    def vocab(self):
        return self.cfg.vocab

    def capturable(self, n_tok):
        """Every step launches a fixed sequence of kernels with no host read in between, so a decode step can be captured."""
        return True

    def alloc_caches(self, n_state_slots, n_token_slots):
        """One cache per layer RUN (a layer inside the looped range has one per pass): the mixer's pages or recurrent state
        and the token shift's carried input; one more entry at the end holds every request's last token (the pair embedding's
        state)."""
        caches = []
        for i, _ in self.runs:
            c = self.layers[i].mixer.alloc_cache(n_state_slots, n_token_slots, self.dtype, self.device)
            c["shift"] = self.layers[i].shift.alloc_cache(n_state_slots, self.device)
            caches.append(c)
        caches.append({"last_token": torch.zeros(n_state_slots, dtype=torch.int32, device=self.device)})
        return caches

    def forward(self, batch, caches, after_layer=None):
        """Logits f32 [len(batch.rows), vocab] of one step's flat batch; advances `caches`.  after_layer(r, x) is called
        with the f32 residual after every layer run (inspection only; what is added before the next pass then comes in a
        pass of its own)."""
        cfg, T, W, eps = self.cfg, batch.ids.numel(), self.cfg.width, self.cfg.eps
        x = torch.empty(T, W, dtype=torch.float32, device=self.device)
        if self.pairs is not None:
            buckets, mul_prev, mul_cur = cfg.bigram
            K.embed_pair(self.embed, self.pairs, batch.ids, cfg.embedding_scale, buckets, mul_prev, mul_cur, caches[-1]["last_token"], batch, x)
        else:
            K.embed_scaled(self.embed, batch.ids, cfg.embedding_scale, x)
        step_of = lambda t: None if t is None else self.loop_step[t]
        i0, t0 = self.runs[0]
        h = K.rms_residual(x, dst=x, add_vec=step_of(t0), next_w=self.layers[i0].norm1, eps=eps, dtype=self.dtype)
        for r, (i, _) in enumerate(self.runs):
            lay = self.layers[i]
            h = lay.shift.forward(h, batch, caches[r]["shift"])
            y, post = lay.mixer.forward(h, batch, caches[r]), lay.norm1b
            if lay.mlp is not None:
                h = K.rms_residual(x, y, dst=x, post_w=post, next_w=lay.norm2, eps=eps)
                y, post = lay.mlp.forward(h), lay.norm2b
            if r + 1 == len(self.runs):
                K.rms_residual(x, y, dst=x, post_w=post, eps=eps)
                if after_layer is not None:
                    after_layer(r, x)
                break
            j, t = self.runs[r + 1]
            if after_layer is None:
                h = K.rms_residual(x, y, dst=x, post_w=post, add_vec=step_of(t), next_w=self.layers[j].norm1, eps=eps)
            else:
                K.rms_residual(x, y, dst=x, post_w=post, eps=eps)
                after_layer(r, x)
                h = K.rms_residual(x, dst=x, add_vec=step_of(t), next_w=self.layers[j].norm1, eps=eps, dtype=self.dtype)
        hn = K.streams_read_norm(x.view(T, 1, W), None, self.final_norm, eps, 0.0, self.dtype, rows=batch.rows)
        return M.linear(hn, self.embed).float()


def random_tensors(cfg: KibotarConfig, seed=0, decay_rank=16):
    """Random bf16-representable weights with activations of order one (throughput runs and tests)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in cfg.tensor_shapes().items():
        shape = tuple(decay_rank if s is None else s for s in shape)
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2", "norm1b", "norm2b", "norm") and len(shape) == 1:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "shift":
            t = torch.rand(shape, generator=g)
        elif leaf == "talk":
            t = torch.eye(shape[0]) + 0.3 * torch.randn(shape, generator=g) / shape[0] ** 0.5
        elif leaf == "step":
            t = 0.1 * torch.randn(shape, generator=g)
        elif leaf == "b":
            t = (1.0 if name.endswith("a2.b") else 0.1) * torch.randn(shape, generator=g)
        elif name in ("embed", "bigram"):
            t = torch.randn(shape, generator=g) / (cfg.embedding_scale if name == "embed" else 1.0)
        else:
            t = torch.randn(shape, generator=g) / shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16)
    return out
