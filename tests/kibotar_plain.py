"""Plain, slow restatement of the Kibotar design in float64 on the CPU: one function per mechanism, whole sequences
at once, no cache, no batching.  TEST INFRASTRUCTURE: it shares no code with the package; the GPU tests compare the
package's kernels, cache and scheduler with it.

Weights are a dict name -> float64 tensor with the checkpoint's names (`embed`, `bigram`, `loop.step`, `l<i>.shift`,
`l<i>.mix.q`, ...); the configuration is the parsed config.json."""
import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


# ---- embedding with a hashed pair table ---------------------------------------------------------------
def pair_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the pair table for every position: a hash of (previous token, token); the extra last row for the first."""
    return [buckets if t == 0 else (tokens[t - 1] * mul_prev + tokens[t] * mul_cur) % buckets for t in range(len(tokens))]


def embed(tokens, table, scale, pair_table, buckets, mul_prev, mul_cur):
    ids = torch.tensor(tokens, dtype=torch.long)
    return table[ids] * scale + pair_table[torch.tensor(pair_rows(tokens, buckets, mul_prev, mul_cur), dtype=torch.long)]


# ---- token shift -----------------------------------------------------------------------------------------
def token_shift(h, mu):
    """h_t + (h_(t-1) - h_t) * mu, with the unshifted predecessor and zeros before the first token."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]])
    return h + (prev - h) * mu


# ---- rotation (halves) -----------------------------------------------------------------------------------
def rotation_frequencies(rot):
    """Angular frequency per rotated pair; long wavelengths are slowed by `factor`, short ones kept, a linear blend between."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = []
        for fi in f:
            wave = 2.0 * math.pi / fi
            if wave < orig / high:
                out.append(fi)
            elif wave > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wave - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = out
    return torch.tensor(f, dtype=F64)


def rotate_halves(x, positions, freq):
    """x [T, heads, d]: entry i < half is paired with entry i + half; the rest passes."""
    half = freq.numel()
    ang = torch.tensor(positions, dtype=F64)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * half:]], dim=-1)


# ---- mixers ----------------------------------------------------------------------------------------------
def gated_linear_attention(h, w, p, m, eps):
    """Per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with a decay per key channel."""
    T, H, dk, dv, tau = h.shape[0], int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["tau"])
    q = (h @ w[p + "q"].T * dk ** -0.5).view(T, H, dk)
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / tau)).view(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = unit_rms(o, eps) * w[p + "norm"]
    return (o.reshape(T, H * dv) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def latent_attention(h, w, p, m, eps):
    """Keys and values of every head decompressed from one normed low-rank latent per token; causal; a gate per head."""
    T, H, dk, dv, R = h.shape[0], int(m["heads"]), int(m["dim"]), int(m["vdim"]), int(m["kv_rank"])
    q = (h @ w[p + "q"].T).view(T, H, dk)
    c = unit_rms(h @ w[p + "dkv"].T, eps) * w[p + "dkv.norm"]
    assert c.shape[1] == R
    k = (c @ w[p + "uk"].T).view(T, H, dk)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):
        s = torch.einsum("hd,jhd->hj", q[i], k[:i + 1]) * float(m["scale"])
        pr = torch.softmax(s, dim=-1)
        out[i] = torch.einsum("hj,jhd->hd", pr, v[:i + 1])
    gate = sigmoid(h @ w[p + "g"].T)               # [T, H]
    return (out * gate[:, :, None]).reshape(T, H * dv) @ w[p + "o"].T


def pooled_window_keys(i, size, pool):
    """What position i sees: (number of pooled blocks, first position of the window)."""
    blocks = max(0, (i - size + 1) // pool) if i - size >= 0 else 0
    return blocks, max(0, i - size + 1)


def pooled_window_attention(h, w, p, m, positions=None):
    """Grouped heads, biased projections, rotation on part of each head, a window of single tokens plus one averaged key
    and value per whole block before it, a softmax whose denominator has one added, weights mixed across heads, a gate
    per output entry."""
    T, H, G, dk, dv = h.shape[0], int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"])
    positions = list(range(T)) if positions is None else positions
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, dk)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, dk)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    if m.get("rot"):
        freq = rotation_frequencies(m["rot"])
        q, k = rotate_halves(q, positions, freq), rotate_halves(k, positions, freq)
    mask = m.get("mask") or {}
    size, pool = int(mask.get("size", 0)), int(mask.get("pool", 0))
    per = H // G
    talk = w[p + "talk"]
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):
        if size > 0:
            nb, lo = pooled_window_keys(i, size, pool) if pool > 0 else (0, max(0, i - size + 1))
        else:
            nb, lo = 0, 0
        keys = [k[b * pool:(b + 1) * pool].mean(0) for b in range(nb)] + [k[j] for j in range(lo, i + 1)]
        vals = [v[b * pool:(b + 1) * pool].mean(0) for b in range(nb)] + [v[j] for j in range(lo, i + 1)]
        kk, vv = torch.stack(keys), torch.stack(vals)                        # [n, G, d]
        kk, vv = kk.repeat_interleave(per, dim=1), vv.repeat_interleave(per, dim=1)      # head h reads group h // per
        s = torch.einsum("hd,jhd->hj", q[i], kk) * float(m["scale"])
        top = max(float(s.max()), 0.0)
        e = torch.exp(s - top)
        pr = e / (math.exp(-top) + e.sum(-1, keepdim=True))                  # the one in the denominator, shifted like the rest
        pr = talk @ pr                                                        # weights of head h <- sum_g talk[h, g] weights of g
        out[i] = torch.einsum("hj,jhd->hd", pr, vv)
    gate = sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[p + "o"].T + w[p + "o.b"]


def dense_ff(h, w, p):
    u = torch.relu(h @ w[p + "up"].T)
    return (u * u) @ w[p + "down"].T


# ---- the model -------------------------------------------------------------------------------------------
def layer_runs(cfg):
    """[(layer, pass number or None)]: the pass number marks the first layer of every pass of the repeated range."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    out = [(i, None) for i in range(a)]
    for t in range(times):
        out += [(i, t if i == a else None) for i in range(a, b)]
    return out + [(i, None) for i in range(b, n)]


def forward(cfg, w, tokens, after_layer=None):
    """Logits [T, vocab] of one whole sequence."""
    eps = float(cfg["norm"]["eps"])
    e = cfg["embedding"]
    bg = e.get("bigram")
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * float(e.get("scale", 1.0))
    if bg:
        rows = pair_rows(tokens, int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"]))
        x = x + w["bigram"][torch.tensor(rows, dtype=torch.long)]
    norm = lambda v, name: unit_rms(v, eps) * w[name]
    for r, (i, start_of_pass) in enumerate(layer_runs(cfg)):
        L, p = cfg["layers"][i], f"l{i}."
        if start_of_pass is not None:
            x = x + w["loop.step"][start_of_pass]
        h = token_shift(norm(x, p + "norm1"), w[p + "shift"])
        if L["type"] == "gla":
            y = gated_linear_attention(h, w, p + "mix.", L["mixer"], eps)
        elif L["type"] == "latent_attention":
            y = latent_attention(h, w, p + "mix.", L["mixer"], eps)
        elif L["type"] == "attention":
            y = pooled_window_attention(h, w, p + "mix.", L["mixer"])
        else:
            raise NotImplementedError(L["type"])
        x = x + norm(y, p + "norm1b")
        if L.get("mlp") is not None:
            x = x + norm(dense_ff(norm(x, p + "norm2"), w, p + "mlp."), p + "norm2b")
        if after_layer is not None:
            after_layer(r, x)
    return norm(x, "final.norm") @ w["embed"].T
