"""Plain, slow restatement of the Fosulix design in float64 on the CPU: one function per mechanism, whole
sequences at once, no cache, no batching.  TEST INFRASTRUCTURE: it shares no code with the package; the GPU tests
compare the package's kernels, cache and scheduler with it.

Weights are a dict name -> float64 tensor with the checkpoint's names (`l<i>.mix.dq`, `l<i>.canon1`, `l<i>.dwa`, ...);
the configuration is the parsed config.json."""
import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


# ---- short convolution over time ------------------------------------------------------------------------
def shifted_sum(h, taps):
    """h [T, C], taps [C, n]: out_t = sum_j taps[:, j] * h_(t - n + 1 + j); nothing before the first token."""
    T, n = h.shape[0], taps.shape[1]
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(n):
            s = t - n + 1 + j
            if s >= 0:
                out[t] += taps[:, j] * h[s]
    return out


# ---- depth-weighted average ------------------------------------------------------------------------------
def depth_average(history, weights):
    """history: list of [T, W] (embedding output, then every layer's result so far); weights: one per entry."""
    assert len(history) == weights.numel()
    return sum(weights[j] * history[j] for j in range(len(history)))


# ---- rotation (neighbouring pairs) -----------------------------------------------------------------------
def rotation_frequencies(rot):
    """Angular frequency per rotated pair and the factor on cos / sin (1 without scaling)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F64), 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])
    turn = lambda t: dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo, hi = max(math.floor(turn(float(sc["fast"]))), 0), min(math.ceil(turn(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate_neighbours(x, rot, first_pos=0):
    """x [T, ..., d]: entries (2i, 2i + 1), i < rot.dims / 2, turn by position * f_i; the rest pass."""
    T, dims = x.shape[0], int(rot["dims"])
    f, mag = rotation_frequencies(rot)
    a = (torch.arange(T, dtype=F64) + first_pos)[:, None] * f[None, :]
    shape = [T] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = (torch.cos(a) * mag).reshape(shape), (torch.sin(a) * mag).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ---- attention through a shared latent -------------------------------------------------------------------
def latent_of(h, w, p, m, eps):
    """The per-token key/value latent and the one rotated key part all heads share: ([T, r], [T, rot_dim])."""
    r = int(m["kv_rank"])
    y = h @ w[p + "dkv"].T
    return unit_rms(y[:, :r], eps) * w[p + "dkv.norm"], rotate_neighbours(y[:, r:], m["rot"])


def latent_attention(h, w, p, m, eps, latent=None):
    """h [T, W].  latent: (c, k_rot) of another layer, or None to form this layer's own.  Returns (out, latent)."""
    T = h.shape[0]
    H, dn, dr, dv = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
    if latent is None:
        latent = latent_of(h, w, p, m, eps)
    c, k_rot = latent
    cq = unit_rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(T, H, dn + dr)
    q_flat, q_rot = q[..., :dn], rotate_neighbours(q[..., dn:], m["rot"])
    k_flat = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j <= i) & (i - j < int(m["mask"]["size"]))
    heads = []
    for a in range(H):
        s = (q_flat[:, a] @ k_flat[:, a].T + q_rot[:, a] @ k_rot.T) * float(m["scale"])
        s = s.masked_fill(~seen, -math.inf)
        e = torch.exp(s - s.max(-1, keepdim=True).values)
        heads.append((e / e.sum(-1, keepdim=True)) @ v[:, a])
    return torch.cat(heads, dim=-1) @ w[p + "o"].T, latent


# ---- gated linear recurrence whose forget gate also writes -------------------------------------------------
def forget_gate(h, w, p):
    """[T, heads * dim] in (lower, 1)."""
    low = w[p + "lower"]
    return low + (1.0 - low) * sigmoid(h @ w[p + "f"].T + w[p + "f.b"])


def tied_gate_recurrence(h, w, p, m, eps):
    T = h.shape[0]
    H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    z = h @ w[p + "q"].T
    q = (z * sigmoid(z)).reshape(T, H, dk)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    f = forget_gate(h, w, p).reshape(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    out = unit_rms(out, eps) * w[p + "norm"]
    return out.reshape(T, H * dv) @ w[p + "o"].T


# ---- routed experts --------------------------------------------------------------------------------------
def choose_experts(scores, top, n_groups, keep):
    """scores [E] -> the chosen expert indices: only the `keep` groups (equal runs of neighbours) whose two largest
    scores sum highest are eligible."""
    E = scores.numel()
    per = E // n_groups
    grouped = scores.reshape(n_groups, per)
    gs = grouped.sort(-1, descending=True).values[:, :2].sum(-1)
    allowed = torch.zeros(n_groups, dtype=torch.bool)
    allowed[gs.topk(keep).indices] = True
    masked = scores.masked_fill(~allowed.repeat_interleave(per), -math.inf)
    return masked.topk(top).indices


def capped_expert(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def routed_experts(h, w, p, mlp):
    r = mlp["router"]
    E, top = int(r["experts"]), int(r["top"])
    groups = r.get("groups") or {"count": 1, "keep": 1}
    scores = sigmoid(h @ w[p + "router"].T)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in choose_experts(scores[t], top, int(groups["count"]), int(groups["keep"])).tolist():
            y = capped_expert(h[t], w[p + f"e{e}.gate"], w[p + f"e{e}.up"], w[p + f"e{e}.down"], float(mlp["expert"]["limit"]))
            out[t] += scores[t, e] * float(r.get("scale", 1.0)) * y
    return out


# ---- the model -------------------------------------------------------------------------------------------
def forward(cj, w, ids, per_layer=None):
    """Logits [T, vocab] of one whole sequence.  per_layer, a list, receives what each layer hands on."""
    eps, mult = float(cj["norm"]["eps"]), float(cj["residual_mult"])
    x = w["embed"][torch.as_tensor(ids, dtype=torch.long)] * float(cj["embedding"]["scale"])
    history, latents = [x], {}
    for i, L in enumerate(cj["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h = unit_rms(x, eps) * w[p + "norm1"]
        h = h + shifted_sum(h, w[p + "canon1"])
        if L["type"] == "latent_attention":
            src = m.get("kv_from")
            y, latents[i] = latent_attention(h, w, p + "mix.", m, eps, None if src is None else latents[int(src)])
        elif L["type"] == "hgrn2":
            y = tied_gate_recurrence(h, w, p + "mix.", m, eps)
        else:
            raise NotImplementedError(L["type"])
        x = x + mult * y
        if L.get("mlp") is not None:
            x = x + mult * routed_experts(unit_rms(x, eps) * w[p + "norm2"], w, p + "mlp.", L["mlp"])
        history.append(x)
        x = depth_average(history, w[p + "dwa"])
        if per_layer is not None:
            per_layer.append(x)
    return (unit_rms(x, eps) * w["final.norm"]) @ w["embed"].T
