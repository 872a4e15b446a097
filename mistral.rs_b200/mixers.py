"""Layer mechanisms built on the sequence-mixer kernels (`seq_ops`), each with its constants as parameters so any
model definition can compose them: multi-stream residuals, Dynamic Tanh norms around a single residual, linear
attention with per-head decay, a stabilised matrix memory (mLSTM), softmax attention over a paged cache (query/key
norm per head or over the whole projection, rotary positions with scaled frequencies, window with kept first tokens,
sink, values that are the keys), attention through a shared low-rank latent (one cached latent per token, which a later
layer may reuse), a linear recurrence whose per-channel forget gate also writes (HGRN2), a short causal convolution added
to a sublayer's input, a Mamba-2 style state-space mixer, two mixers side by side, dense GLU / plain and routed-expert
feed-forwards (softmax or sigmoid routing, groups scored by their best or their few best experts, plain or capped GLU),
a token shift (a sublayer's input blended with its predecessor's), gated linear attention with a decay per key channel,
attention whose far past is seen as averaged blocks and whose softmax weights are mixed across heads, output gates per
entry or per head.

A mechanism owns its device weights and declares the per-layer cache it needs (`alloc_cache`): token-indexed pages
(sized by the engine's block pool) and / or per-request state slots (sized by the engine's slot pool).  `forward`
takes the activation rows of one step's flat batch (`engine.StepBatch`) — prompt portions and single decoded tokens
side by side — and advances that cache.  Dense matrix products are plain library GEMMs (`torch.nn.functional.linear`,
cuBLAS); everything between them is this package's CUDA."""
import torch
import torch.nn.functional as F

from . import seq_ops as K


def linear(x, w):
    return F.linear(x, w)


class StreamResidual:
    """Hyper-connections: `n_streams` f32 copies of the residual; a sublayer reads sum_s w_in[s] x_s and writes
    x_r <- sum_s w_mix[s, r] x_s + w_out[r] y."""

    def __init__(self, w_in, w_out, w_mix):
        self.w_in, self.w_out, self.w_mix = w_in, w_out, w_mix


class LinearAttentionMixer:
    """q, k, v = act(W h) per head; S_t = decay_h S_(t-1) + k_t v_t^T; o_t = S_t^T q_t; RMS norm over the concatenated
    heads, output gate sigmoid(W_g h), output projection."""

    def __init__(self, w_qkvg, w_o, norm_w, decay, heads, dk, dv, eps, act=K.ACT_SILU):
        self.w_qkvg, self.w_o, self.norm_w, self.decay = w_qkvg, w_o, norm_w, decay
        self.heads, self.dk, self.dv, self.eps, self.act = heads, dk, dv, eps, act

    def alloc_cache(self, n_slots, n_token_slots, dtype, device):
        return {"state": torch.zeros(n_slots, self.heads, self.dk, self.dv, dtype=torch.float32, device=device)}

    def forward(self, h, batch, cache):
        H, dk, dv = self.heads, self.dk, self.dv
        y = linear(h, self.w_qkvg)                                         # [T, 2 H dk + 2 H dv]: q | k | v | g
        K.activate_cols(y, 0, 2 * H * dk + H * dv, self.act)                # once, not once per state tile inside the scan
        o = K.linear_scan(y, 0, y, H * dk, y, 2 * H * dk, H, H, dk, dv, cache["state"], batch, decay_head=self.decay)
        on = torch.empty(h.shape[0], H * dv, dtype=h.dtype, device=h.device)
        K.gated_group_norm(o, y, 2 * H * dk + H * dv, self.norm_w, 1, self.eps, K.ACT_SIGMOID, False, on)
        return linear(on, self.w_o)


class TanhNorm:
    """Dynamic Tanh: tanh(alpha z) * weight + bias — a norm that computes no statistics.  `t` is what the kernels take."""

    def __init__(self, alpha, weight, bias):
        self.t = (alpha, weight, bias)


class Rotation:
    """Rotary positions on the first `dims` entries of every head, frequency base^(-2i/dims) for pair i.  Which two entries
    make pair i, (i, i + dims / 2) or the neighbours (2i, 2i + 1), is the choice of the kernel that applies the table.
    `scaling` (YaRN: factor, original, fast, slow) divides the slow frequencies by `factor` along a linear ramp between
    the pair indices at which `original` positions make `fast` and `slow` turns, and multiplies cos and sin by
    0.1 ln(factor) + 1; with the keys factor, original, low, high it is the wavelength rule instead (no magnitude).  Frequencies are formed in double on the host; the table of a step (one per distinct
    rotation, shared by the layers that use it) comes from `seq_ops.rotation_table`."""

    def __init__(self, dims, base, scaling, device):
        import math
        dims, base = int(dims), float(base)
        if dims < 2 or dims % 2:
            raise ValueError("rotated dimensions come in pairs")
        freq, self.mag = [base ** (-2.0 * i / dims) for i in range(dims // 2)], 1.0
        if scaling and "low" in scaling:
            # by wavelength (the rule of Llama 3.1): shorter than original / high: kept; longer than original / low: divided by
            # factor; between, a linear blend in original / wavelength
            factor, orig, low, high = (float(scaling[k]) for k in ("factor", "original", "low", "high"))
            scaled = []
            for f in freq:
                wave = 2.0 * math.pi / f
                if wave < orig / high:
                    scaled.append(f)
                elif wave > orig / low:
                    scaled.append(f / factor)
                else:
                    t = (orig / wave - low) / (high - low)
                    scaled.append((1.0 - t) * f / factor + t * f)
            freq = scaled
        elif scaling:
            factor, orig = float(scaling["factor"]), float(scaling["original"])
            turn = lambda t: dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
            lo, hi = max(math.floor(turn(float(scaling["fast"]))), 0), min(math.ceil(turn(float(scaling["slow"]))), dims - 1)
            ramp = [min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(dims // 2)]
            freq = [f / factor * r + f * (1.0 - r) for f, r in zip(freq, ramp)]
            self.mag = 0.1 * math.log(factor) + 1.0
        self.dims = dims
        self.key = (dims, base, tuple(sorted((k, float(v)) for k, v in scaling.items())) if scaling else None)
        self.freq = torch.tensor(freq, dtype=torch.float64, device=device)

    def table(self, batch):
        tables = batch.__dict__.setdefault("_rotation_tables", {})
        if self.key not in tables:
            tables[self.key] = K.rotation_table(batch.pos_of_tok, self.freq, self.mag)
        return tables[self.key]


class WindowAttention:
    """Grouped-query softmax attention over pages.  Queries and keys: RMS norm per head with weights shared by the
    heads (`norm_mode` QK_NORM_HEAD), over the whole projection at once (QK_NORM_WHOLE) or none; then `rotation` (None:
    scores carry no position).  Scores are scaled by a given constant.  Position i sees j <= i with i - j < `window`
    (0: full causal) or j < `keep_first`; `sink` [heads] adds exp(sink) to the softmax denominator.  With
    `values_from_keys` there is no value projection: the values are the keys as projected, before norm and rotation.

    `pool` > 0 (needs a window and the page size): the positions before the window are seen block-wise — one key and one
    value per block of `pool` positions that lies wholly before the window, each the mean of the block's cached keys /
    values; tokens that left the window while their block is incomplete from the query's point of view are not seen.  The
    means live behind the token rows of the same cache tensors and are formed when a block's last position is stored.

    `talk` [heads, heads] f32: the softmax weights are mixed across heads afterwards, w'_h = sum_g talk[h, g] w_g, and head h
    applies w'_h to the values of its own key/value head (a sink's share is not mixed).  Computed through linearity: the
    attention kernel applies every head's weights to all value heads in f32, `seq_ops.mix_heads` sums over g."""

    def __init__(self, heads, kv_heads, dk, dv, scale, window, q_norm_w, k_norm_w, eps, norm_mode=K.QK_NORM_HEAD, rotation=None,
                 keep_first=0, sink=None, values_from_keys=False, pool=0, talk=None, page_size=None):
        if pool > 0 and (window <= 0 or keep_first > 0 or not page_size):
            raise ValueError("averaged blocks need a window, no kept first tokens, and the page size")
        self.pool, self.talk, self.pool_page_size, self.pool_base = int(pool), talk, page_size, 0
        if values_from_keys and dk != dv:
            raise ValueError("values that are the keys need equal key and value head sizes")
        if heads % kv_heads:
            raise ValueError("query heads must be a multiple of key/value heads")
        self.heads, self.kv_heads, self.dk, self.dv = heads, kv_heads, dk, dv
        self.scale, self.window, self.q_norm_w, self.k_norm_w, self.eps = scale, window, q_norm_w, k_norm_w, eps
        self.norm_mode = norm_mode if q_norm_w is not None else K.QK_NORM_NONE
        self.rotation, self.keep_first, self.sink, self.values_from_keys = rotation, keep_first, sink, values_from_keys

    @property
    def proj_cols(self):
        return self.heads * self.dk + self.kv_heads * self.dk + (0 if self.values_from_keys else self.kv_heads * self.dv)

    def alloc_cache(self, n_slots, n_token_slots, dtype, device):
        rows = n_token_slots
        if self.pool > 0:                      # the averaged blocks' rows follow the token rows
            self.pool_base = n_token_slots
            rows += K.pool_rows(n_token_slots, self.pool_page_size, self.pool)
        return {"k": torch.zeros(rows, self.kv_heads, self.dk, dtype=dtype, device=device),
                "v": torch.zeros(rows, self.kv_heads, self.dv, dtype=dtype, device=device)}

    def attend(self, y, col0, batch, cache, page_size, out, out_col=0, out_scale=1.0, gate_col=None, gate_act=K.ACT_SIGMOID):
        """y holds q | k | v (q | k when the values are the keys) from column col0; writes heads * dv columns of `out`
        from out_col.  Keys and values of the new tokens are normed, rotated and stored first.  Long portions (32 tokens
        or more) run on tensor cores when they fit (bf16, equal head sizes of 64 or 128, 16-byte aligned rows): when every
        one of them starts its sequence and the layer has neither sink nor kept first tokens, on the package's prompt
        kernels over the fresh q / k / v; otherwise — sinks, kept tokens, portions that continue a sequence — on the
        sequence library's prompt kernel, which reads keys and values from the pages.  Every other token (short portions,
        decoded tokens, other head sizes, f32) runs on the (token, head) kernel over the pages, and so does every token of a
        layer with averaged blocks or mixed heads.  gate_col: columns of y (heads * dv of them) whose `gate_act` multiplies the
        result entry by entry."""
        kc = col0 + self.heads * self.dk
        vc = None if self.values_from_keys else kc + self.kv_heads * self.dk
        cos_sin = self.rotation.table(batch) if self.rotation is not None else None
        K.attention_prepare(y, col0, kc, vc, self.norm_mode, self.q_norm_w, self.k_norm_w, self.eps, self.heads, self.kv_heads, self.dk,
                            self.dv, cache["k"], cache["v"], batch.slot_of_tok, cos_sin, self.rotation.dims if cos_sin is not None else 0)
        if self.pool > 0:
            if page_size != self.pool_page_size or cache["k"].shape[0] <= self.pool_base:
                raise ValueError("the cache was not made for this layer's averaged blocks")
            K.pool_blocks(cache["k"], cache["v"], self.kv_heads * self.dk, self.kv_heads * self.dv, self.pool, self.pool_base, batch, page_size)
        if self.pool > 0 or self.talk is not None:
            self._attend_general(y, col0, batch, cache, page_size, out, out_col, out_scale, gate_col, gate_act)
            return
        self._attend_plain(y, col0, kc, vc, batch, cache, page_size, out, out_col, out_scale)
        if gate_col is not None:
            K.gate_cols(out[:, out_col:], y, gate_col, self.heads * self.dv, 1, gate_act)

    def _attend_general(self, y, col0, batch, cache, page_size, out, out_col, out_scale, gate_col, gate_act):
        """Averaged blocks and / or mixed heads.  Long portions take the sequence library's tensor-core prompt kernel when they
        fit (bf16, equal head sizes of 64 or 128, aligned rows) — with mixed heads once per value head, every head's weights on
        that head's values; every other token takes the (token, head) kernel, which reads a row's value heads side by side."""
        H, G, dv = self.heads, self.kv_heads, self.dv
        mixed = self.talk is not None
        res = torch.empty(y.shape[0], H * G * dv, dtype=torch.float32, device=y.device) if mixed else out      # mixed: head g's weights on every value head
        res_col = 0 if mixed else out_col
        tok_index = None
        fits = y.dtype == torch.bfloat16 and self.dk == dv and dv in (64, 128) and not self.values_from_keys and \
            all(v % 8 == 0 for v in (y.stride(0), col0, res.stride(0), res_col))
        if batch.long and fits:
            K.prompt_attention(y, col0, cache["k"], cache["v"], batch, page_size, H, G, dv, self.scale, self.window, self.keep_first, self.sink, res,
                               res_col, pool=self.pool, pool_base=self.pool_base, every_value_head=mixed)
            if out_scale != 1.0:
                for row0, rows, _, _ in batch.long:
                    K.scale_rows(res, row0, rows, res_col, res.shape[1] if mixed else H * dv, out_scale)
            tok_index = batch.short_tok
        if tok_index is None or tok_index.numel() > 0:
            if mixed:          # as many value heads per launch as the kernel's vector path takes (512 value columns)
                per_call = max(1, 512 // dv)
                for g0 in range(0, G, per_call):
                    n = min(per_call, G - g0)
                    K.paged_attention(y, col0, cache["k"], cache["v"], H, G, self.dk, n * dv, self.scale, self.window, self.keep_first, self.sink,
                                      batch, page_size, res, g0 * dv, out_scale, tok_index, v_row=G * dv, pool=self.pool, pool_base=self.pool_base,
                                      v_shared=True, v_col=g0 * dv, out_head=G * dv)
            else:
                K.paged_attention(y, col0, cache["k"], cache["v"], H, G, self.dk, dv, self.scale, self.window, self.keep_first, self.sink, batch,
                                  page_size, out, out_col, out_scale, tok_index, pool=self.pool, pool_base=self.pool_base)
        if mixed:
            K.mix_heads(res, self.talk, H, G, dv, out[:, out_col:], y if gate_col is not None else None, gate_col or 0, gate_act)
        elif gate_col is not None:
            K.gate_cols(out[:, out_col:], y, gate_col, H * dv, 1, gate_act)

    def _attend_plain(self, y, col0, kc, vc, batch, cache, page_size, out, out_col, out_scale):
        tok_index = None
        aligned = all(v % 8 == 0 for v in (y.stride(0), col0, out.stride(0), out_col))
        if batch.long and y.dtype == torch.bfloat16 and self.dk == self.dv and self.dk in (64, 128) and aligned:
            plain = self.sink is None and self.keep_first == 0 and vc is not None       # what the package's prompt kernels know
            if plain and len(batch.fresh) == len(batch.long):
                for row0, rows in batch.fresh:
                    K.fresh_prompt_attention(y, row0, rows, col0, kc, vc, self.heads, self.kv_heads, self.dk, self.scale, self.window, out, out_col)
            else:
                K.prompt_attention(y, col0, cache["k"], cache["v"], batch, page_size, self.heads, self.kv_heads, self.dk, self.scale, self.window,
                                   self.keep_first, self.sink, out, out_col)
            if out_scale != 1.0:
                for row0, rows, _, _ in batch.long:
                    K.scale_rows(out, row0, rows, out_col, self.heads * self.dv, out_scale)
            tok_index = batch.short_tok
            if tok_index.numel() == 0:
                return
        K.paged_attention(y, col0, cache["k"], cache["v"], self.heads, self.kv_heads, self.dk, self.dv, self.scale, self.window,
                          self.keep_first, self.sink, batch, page_size, out, out_col, out_scale, tok_index)


class InputConvolution:
    """h <- h + conv(h): a causal convolution over time on every channel, conv(h)_t = sum_j taps[:, j] h_(t - n + 1 + j), added
    to its own input before a sublayer reads it.  The last n - 1 inputs of every request are state (one slot each); the
    identity rides on the last tap, so this is the package's short-convolution kernel with f32 taps."""

    def __init__(self, taps):
        w = taps.to(torch.float32).clone()
        w[:, -1] += 1.0
        self.taps = w.contiguous()

    def alloc_cache(self, n_slots, device):
        return torch.zeros(n_slots, max(self.taps.shape[1] - 1, 1), self.taps.shape[0], dtype=torch.float32, device=device)

    def forward(self, h, batch, state):
        return K.causal_conv(h, 0, self.taps.shape[0], self.taps, None, K.ACT_NONE, state, batch)


class TokenShift(InputConvolution):
    """h <- h + (h_prev - h) * mu: every channel of a sublayer's input is blended with the same channel of the previous
    token's (unshifted) input, zeros before a sequence's first token.  It is the two-tap case of the input convolution,
    h + (mu * h_prev - mu * h); the previous input of every request is state (one slot each)."""

    def __init__(self, mu):
        mu = mu.to(torch.float32).reshape(-1, 1)
        super().__init__(torch.cat([mu, -mu], dim=1))


class LatentAttentionMixer:
    """Multi-head latent attention.  Queries: c_q = rms_norm(W_dq h) w, q = W_uq c_q, per head [dn plain | dr rotated].
    Keys / values: W_dkv h = [kv_rank | dr]; c = rms_norm(first part) w is the latent, the last dr entries (rotated, not
    normed) are one key part all heads share; k_h = [W_uk,h c | shared part], v_h = W_uv,h c.  Only c and the shared part
    are cached (one row of kv_rank + dr per token).  Rotation turns neighbouring pairs.  Scores are scaled by a given
    constant; position i sees j with 0 <= i - j < window (0: all).

    Computed in the absorbed form: a head's query becomes [W_uk,h^T q_plain | q_rot] (size kv_rank + dr), attention runs
    over the cached rows as one key/value head whose values are the rows' first kv_rank columns, and W_uv,h maps the
    result to the head's output.  In bf16 every sequence of a step, a prompt portion or a single decoded token, runs on the
    tensor-core latent kernel (all heads of a token share one fetched key tile); f32, and sizes the kernel does not take,
    run on the (token, head) kernel over the pages.  `shares`: this mixer has no W_dkv and reads the cache another layer fills.

    When every sequence of a step starts in it with a long portion (whole prompts) and the sizes allow (bf16, no rotated part,
    dn = dv of 64 or 128, at least DECOMPRESS_MIN_TOKENS tokens), keys and values ARE decompressed, for this step only: two
    products turn the step's normed latents into per-head keys and values, and the plain tensor-core prompt kernel runs over
    these dense rows — dn + dv multiply-adds per (query, key, head) instead of 2 kv_rank.  The cache still holds only latents.

    q_rank 0: there is no query latent — w_down's first heads * (dn + dr) rows are the query projection itself (w_uq and
    q_norm_w are None).  dr 0 with rotation None: no rotated part, scores carry no position.  `head_gate`: w_down ends with
    `heads` more rows, and head h's output is multiplied by that activation of row h's product (a gate per head)."""

    def __init__(self, w_down, w_uq, w_uk, w_uv, w_o, q_norm_w, kv_norm_w, heads, dn, dr, dv, q_rank, kv_rank, scale, window, rotation, eps,
                 page_size, shares=False, head_gate=None):
        self.head_gate = head_gate
        self.w_down, self.w_uq, self.w_o, self.q_norm_w, self.kv_norm_w = w_down, w_uq, w_o, q_norm_w, kv_norm_w
        self.w_uk_rows, self.w_uv_rows = w_uk, w_uv                      # [H dn, r] / [H dv, r]: the decompressing products
        self.w_uk = w_uk.view(heads, dn, kv_rank)                       # [H][dn][r]: q_plain,h @ w_uk[h] = W_uk,h^T q_plain,h
        self.w_uv_t = w_uv.view(heads, dv, kv_rank).transpose(1, 2)     # [H][r][dv]
        self.heads, self.dn, self.dr, self.dv, self.q_rank, self.kv_rank = heads, dn, dr, dv, q_rank, kv_rank
        self.scale, self.window, self.rotation, self.eps, self.page_size, self.shares = scale, window, rotation, eps, page_size, shares
        self.row = kv_rank + dr

    def alloc_cache(self, n_slots, n_token_slots, dtype, device):
        if self.shares:
            return {}
        row = -(-self.row // 8) * 8            # rows start on 16-byte boundaries
        return {"latent": torch.zeros(n_token_slots, row, dtype=dtype, device=device)}

    DECOMPRESS_MIN_TOKENS = 256

    def decompresses(self, h, batch):
        """True when this step's keys and values are decompressed (see the class text)."""
        return (h.dtype == torch.bfloat16 and not self.shares and self.dr == 0 and self.dn == self.dv and self.dv in (64, 128) and
                self.kv_rank % 8 == 0 and self.w_down.shape[0] % 8 == 0 and batch.n_seq > 0 and len(batch.long) == batch.n_seq and
                all(past == 0 for _, _, past, _ in batch.long) and h.shape[0] >= self.DECOMPRESS_MIN_TOKENS)

    def forward(self, h, batch, cache):
        T, H, dn, dr, R = h.shape[0], self.heads, self.dn, self.dr, self.kv_rank
        latent = cache["latent"]
        if self.decompresses(h, batch):
            y = linear(h, self.w_down)
            q_cols = self.q_rank if self.q_rank > 0 else H * dn
            c = torch.empty(T, R, dtype=h.dtype, device=h.device)
            cq = torch.empty(T, self.q_rank, dtype=h.dtype, device=h.device) if self.q_rank > 0 else None
            K.latent_prepare(y, 0, self.q_rank, self.q_norm_w, cq, q_cols, R, 0, 0, self.kv_norm_w, None, self.eps, latent, batch.slot_of_tok, kv_out=c)
            q2 = linear(cq, self.w_uq) if self.q_rank > 0 else y
            out = torch.empty(T, H * self.dv, dtype=h.dtype, device=h.device)
            K.dense_prompt_attention(q2, 0, linear(c, self.w_uk_rows), linear(c, self.w_uv_rows), batch, H, H, self.dv, self.scale, self.window,
                                     None, out)
            if self.head_gate is not None:
                K.gate_cols(out, y, q_cols + R, H * self.dv, self.dv, self.head_gate)
            return linear(out, self.w_o)
        cos_sin = self.rotation.table(batch) if self.rotation is not None else None
        rot_dims = self.rotation.dims if self.rotation is not None else 0
        y = linear(h, self.w_down)                                           # query latent (or queries) | (key/value latent | shared key part) | (gates)
        q_cols = self.q_rank if self.q_rank > 0 else H * (dn + dr)
        if self.q_rank > 0:
            cq = torch.empty(T, self.q_rank, dtype=h.dtype, device=h.device)
            K.latent_prepare(y, 0, self.q_rank, self.q_norm_w, cq, q_cols, 0 if self.shares else R, dr, rot_dims, self.kv_norm_w, cos_sin,
                             self.eps, latent, batch.slot_of_tok)
            q2 = linear(cq, self.w_uq)
        else:
            if not self.shares:
                K.latent_prepare(y, 0, 0, None, None, q_cols, R, dr, rot_dims, self.kv_norm_w, cos_sin, self.eps, latent, batch.slot_of_tok)
            q2 = y[:, :q_cols]
        q = q2.unflatten(1, (H, dn + dr))
        qa = torch.empty(T, H, self.row, dtype=h.dtype, device=h.device)      # the absorbed queries
        torch.bmm(q[:, :, :dn].transpose(0, 1), self.w_uk, out=qa[:, :, :R].transpose(0, 1))
        if dr > 0:
            K.rotate_pairs(q2, dn, dn + dr, qa.view(T, -1), R, self.row, H, dr, rot_dims, cos_sin)
        o = torch.empty(T, H, R, dtype=h.dtype, device=h.device)
        if h.dtype == torch.bfloat16 and K.latent_attention_fits(R, dr) and latent.stride(0) % 8 == 0:
            K.latent_prompt_attention(qa.view(T, -1), latent, H, R, dr, self.scale, self.window, batch, self.page_size, o.view(T, -1))
        else:
            K.latent_attention(qa.view(T, -1), latent, H, R, dr, self.scale, self.window, batch, self.page_size, o.view(T, -1))
        out = torch.empty(T, H, self.dv, dtype=h.dtype, device=h.device)
        torch.bmm(o.transpose(0, 1), self.w_uv_t, out=out.transpose(0, 1))
        if self.head_gate is not None:
            gate_col = q_cols + (0 if self.shares else R + dr)
            K.gate_cols(out.view(T, H * self.dv), y, gate_col, H * self.dv, self.dv, self.head_gate)
        return linear(out.view(T, H * self.dv), self.w_o)


class TiedGateMixer:
    """HGRN2: linear attention whose forget gate also decides what is written.  q = silu(W_q h), v = W_v h, per head and
    channel f = lower + (1 - lower) sigmoid(W_f h + b) in f32; S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t;
    every head's o is RMS-normed over its value size with weights shared by the heads; output projection.  The
    recurrence is the package's linear scan with a decay per state row, whose key is the decay's complement."""

    def __init__(self, w_qfv, f_bias, lower, w_o, norm_w, heads, dk, dv, eps):
        self.w_qfv, self.f_bias, self.lower, self.w_o = w_qfv, f_bias, lower, w_o
        self.norm_w = norm_w.repeat(heads).contiguous()            # the group norm takes one weight per column
        self.heads, self.dk, self.dv, self.eps = heads, dk, dv, eps

    def alloc_cache(self, n_slots, n_token_slots, dtype, device):
        return {"state": torch.zeros(n_slots, self.heads, self.dk, self.dv, dtype=torch.float32, device=device)}

    def forward(self, h, batch, cache):
        H, dk, dv = self.heads, self.dk, self.dv
        y = linear(h, self.w_qfv)                                          # [T, 2 H dk + H dv]: q | f | v
        K.activate_cols(y, 0, H * dk, K.ACT_SILU)
        f = K.bounded_gate(y, H * dk, H * dk, self.f_bias, self.lower)
        o = K.linear_scan(y, 0, None, 0, y, 2 * H * dk, H, H, dk, dv, cache["state"], batch, decay_vec=f)
        on = torch.empty(h.shape[0], H * dv, dtype=h.dtype, device=h.device)
        K.gated_group_norm(o, None, 0, self.norm_w, H, self.eps, K.ACT_NONE, False, on)
        return linear(on, self.w_o)


class GatedLinearAttentionMixer:
    """Linear attention with a decay per key channel: q = W_q h * q_scale, k = W_k h, v = W_v h; per head and key channel
    alpha = sigmoid(W_a2 (W_a1 h) + b)^(1 / tau), formed in f32 from the low-rank projection's output; S_t = diag(alpha_t)
    S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; every head's o is RMS-normed over its value size with weights shared by the heads,
    multiplied by silu(W_g h), and projected.  The recurrence is the package's linear scan with a decay per state row and keys
    of their own.  w_in rows: q | k | v | g | a1."""

    def __init__(self, w_in, w_a2, a_bias, tau, w_o, norm_w, heads, dk, dv, q_scale, eps, low_rank):
        self.w_in, self.w_a2, self.a_bias, self.inv_tau, self.w_o = w_in, w_a2, a_bias, 1.0 / float(tau), w_o
        self.norm_w = norm_w.repeat(heads).contiguous()            # the group norm takes one weight per column
        self.heads, self.dk, self.dv, self.q_scale, self.eps, self.low_rank = heads, dk, dv, float(q_scale), eps, low_rank

    def alloc_cache(self, n_slots, n_token_slots, dtype, device):
        return {"state": torch.zeros(n_slots, self.heads, self.dk, self.dv, dtype=torch.float32, device=device)}

    def forward(self, h, batch, cache):
        H, dk, dv = self.heads, self.dk, self.dv
        y = linear(h, self.w_in)                                           # [T, 2 H dk + 2 H dv + r]: q | k | v | g | a1
        g_col = 2 * H * dk + H * dv
        z = linear(y[:, g_col + H * dv:g_col + H * dv + self.low_rank], self.w_a2)
        alpha = K.power_gate(z, 0, H * dk, self.a_bias, self.inv_tau)
        o = K.linear_scan(y, 0, y, H * dk, y, 2 * H * dk, H, H, dk, dv, cache["state"], batch, decay_vec=alpha, q_scale=self.q_scale)
        on = torch.empty(h.shape[0], H * dv, dtype=h.dtype, device=h.device)
        K.gated_group_norm(o, y, g_col, self.norm_w, H, self.eps, K.ACT_SILU, False, on)
        return linear(on, self.w_o)


class AttentionMixer:
    """A `WindowAttention` with its own projections: one input GEMM for q | k | v (optionally biased), attention,
    output projection (optionally biased).  `gate_act`: w_in has heads * dv more rows after q | k | v, and the attention's
    result is multiplied entry by entry with that activation of them before the output projection."""

    def __init__(self, attn: WindowAttention, w_in, w_out, page_size, b_in=None, b_out=None, gate_act=None):
        self.attn, self.w_in, self.w_out, self.b_in, self.b_out, self.page_size = attn, w_in, w_out, b_in, b_out, page_size
        self.gate_act = gate_act

    def alloc_cache(self, n_slots, n_token_slots, dtype, device):
        return self.attn.alloc_cache(n_slots, n_token_slots, dtype, device)

    def forward(self, h, batch, cache):
        y = F.linear(h, self.w_in, self.b_in)
        o = torch.empty(h.shape[0], self.attn.heads * self.attn.dv, dtype=h.dtype, device=h.device)
        if self.gate_act is None:
            self.attn.attend(y, 0, batch, cache, self.page_size, o)
        else:
            self.attn.attend(y, 0, batch, cache, self.page_size, o, gate_col=self.attn.proj_cols, gate_act=self.gate_act)
        return F.linear(o, self.w_out, self.b_out)


class MatrixMemoryMixer:
    """Stabilised matrix memory (mLSTM): per head S_t = keep_t S_(t-1) + take_t k_t v_t^T and n_t likewise with k_t alone,
    keep / take from capped log gates and their running maximum m (from 0); y_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t))
    + 1e-6) with q scaled by dk^(-1/2); unit RMS per head, weight, output gate sigmoid(W_g h), output projection.
    The recurrence is the package's linear scan with per-token decay and input scale; n is the state's extra column
    under a value that is constantly 1.  Gate pre-activations are an f32 product."""

    def __init__(self, w_qkvg, w_gates, b_gates, w_o, norm_w, heads, dk, dv, cap, eps):
        self.w_qkvg, self.w_gates, self.b_gates, self.w_o, self.norm_w = w_qkvg, w_gates, b_gates, w_o, norm_w
        self.heads, self.dk, self.dv, self.cap, self.eps = heads, dk, dv, cap, eps
        self.dvp = -(-(dv + 1) // 8) * 8            # values + the ones column, padded to whole 16-byte groups

    def alloc_cache(self, n_slots, n_token_slots, dtype, device):
        return {"state": torch.zeros(n_slots, self.heads, self.dk, self.dvp, dtype=torch.float32, device=device),
                "m": torch.zeros(n_slots, self.heads, dtype=torch.float32, device=device)}

    def forward(self, h, batch, cache):
        H, dk, dv = self.heads, self.dk, self.dv
        y = linear(h, self.w_qkvg)                                         # [T, 2 H dk + 2 H dv]: q | k | v | g
        raw = torch.addmm(self.b_gates, h.float(), self.w_gates.t())        # [T, 2 H]: input gates | forget gates
        keep, take, m_tok = K.mlstm_gates(raw, H, self.cap, cache["m"], batch)
        vaug = K.append_ones(y, 2 * H * dk, H, dv, self.dvp)
        o = K.linear_scan(y, 0, y, H * dk, vaug, 0, H, H, dk, self.dvp, cache["state"], batch, decay_tok=keep, scale_tok=take)
        on = K.mlstm_out_norm(o, self.dvp, m_tok, dk ** -0.5, y, 2 * H * dk + H * dv, self.norm_w, self.eps, H, dv, h.dtype)
        return linear(on, self.w_o)


class StateSpaceMixer:
    """Mamba-2 (state-space duality) core: the input projection's columns are z | x | B | C | dt; x, B, C pass a short
    causal convolution and silu; dt = softplus(dt + bias); per head S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T,
    y_t = S_t^T C_t + D x_t; y * silu(z) is RMS-normed in `norm_groups` parts."""

    def __init__(self, heads, dv, n_state, groups, norm_groups, conv_w, conv_b, dt_bias, a_log, d_skip, norm_w, eps):
        self.heads, self.dv, self.n_state, self.groups, self.norm_groups = heads, dv, n_state, groups, norm_groups
        self.conv_w, self.conv_b, self.dt_bias, self.a_log, self.d_skip, self.norm_w, self.eps = conv_w, conv_b, dt_bias, a_log, d_skip, norm_w, eps
        self.inner = heads * dv
        self.conv_channels = self.inner + 2 * groups * n_state

    @property
    def proj_cols(self):
        return 2 * self.inner + 2 * self.groups * self.n_state + self.heads

    def alloc_cache(self, n_slots, n_token_slots, dtype, device):
        taps = self.conv_w.shape[1]
        return {"state": torch.zeros(n_slots, self.heads, self.n_state, self.dv, dtype=torch.float32, device=device),
                "conv": torch.zeros(n_slots, max(taps - 1, 1), self.conv_channels, dtype=torch.float32, device=device)}

    def mix(self, y, col0, batch, cache, out, out_col=0, out_scale=1.0):
        """y holds z | xBC | dt from column col0; writes `inner` columns of `out` from out_col."""
        inner, GN = self.inner, self.groups * self.n_state
        xbc = K.causal_conv(y, col0 + inner, self.conv_channels, self.conv_w, self.conv_b, K.ACT_SILU, cache["conv"], batch)
        step, decay = K.ssm_steps(y, col0 + 2 * inner + 2 * GN, self.dt_bias, self.a_log)
        o = K.linear_scan(xbc, inner + GN, xbc, inner, xbc, 0, self.heads, self.groups, self.n_state, self.dv, cache["state"], batch,
                          decay_tok=decay, scale_tok=step, skip=self.d_skip)
        K.gated_group_norm(o, y, col0, self.norm_w, self.norm_groups, self.eps, K.ACT_SILU, True, out, out_col, out_scale)


class ParallelMixer:
    """Windowed attention and a state-space mixer reading the same input; result = left_scale * attention branch +
    right_scale * state-space branch.  One input GEMM feeds both; the scaled branch outputs sit side by side so one
    output GEMM over [W_o_left | W_o_right] sums them in its f32 accumulator."""

    def __init__(self, attn: WindowAttention, ssm: StateSpaceMixer, w_in, w_out, left_scale, right_scale, page_size):
        self.attn, self.ssm, self.w_in, self.w_out = attn, ssm, w_in, w_out
        self.left_scale, self.right_scale, self.page_size = left_scale, right_scale, page_size

    def alloc_cache(self, n_slots, n_token_slots, dtype, device):
        c = self.attn.alloc_cache(n_slots, n_token_slots, dtype, device)
        c.update(self.ssm.alloc_cache(n_slots, n_token_slots, dtype, device))
        return c

    def forward(self, h, batch, cache):
        y = linear(h, self.w_in)                                          # q | k | v | z | xBC | dt
        a_cols = self.attn.heads * self.attn.dv
        both = torch.empty(h.shape[0], a_cols + self.ssm.inner, dtype=h.dtype, device=h.device)
        self.attn.attend(y, 0, batch, cache, self.page_size, both, 0, self.left_scale)
        self.ssm.mix(y, self.attn.proj_cols, batch, cache, both, a_cols, self.right_scale)
        return linear(both, self.w_out)


class DenseGLU:
    """down(act(gate h) * up h) with gate and up as one GEMM."""

    def __init__(self, w_gate_up, w_down, act):
        self.w_gate_up, self.w_down, self.act = w_gate_up, w_down, act

    def forward(self, h):
        return linear(K.glu_split(linear(h, self.w_gate_up), self.act), self.w_down)


class DenseMLP:
    """down(act(up h)): a feed-forward without a gate."""

    def __init__(self, w_up, w_down, act):
        self.w_up, self.w_down, self.act = w_up, w_down, act

    def hidden(self, h):
        u = linear(h, self.w_up)
        K.activate_cols(u, 0, u.shape[1], self.act)
        return u

    def forward(self, h):
        return linear(self.hidden(h), self.w_down)

    def forward_added_to(self, h, other):
        """other + down(act(up h)): the sum forms in the product's f32 accumulator."""
        return torch.addmm(other, self.hidden(h), self.w_down.t())


class RoutedExperts:
    """Router logits in f32.  Rule "grouped_softmax": softmax over all experts, a choice-only bias, group-limited top-k,
    weights = the scores (optionally renormalised).  Rule "grouped_sigmoid": the same with scores = sigmoid(logit).  In both
    a group's score is the sum of its `group_top` largest choices and the weights are multiplied by `weight_scale`.  Rule
    "top_softmax": the largest logits, weights = softmax over the chosen logits alone.  `act`: an activation code or a
    `seq_ops.GluRule` (how gate and up are joined).  Experts are GLU feed-forwards (`gated`: w_up holds gate | up rows) or plain down(act(up h)); a
    `shared` feed-forward, when given, runs for every token and is added.  Few (token, expert) pairs: two
    weight-streaming kernels.  Many: rows sorted by expert, one GEMM pair per expert that has rows (the per-expert row
    counts cross to the host once per layer), weighted combine in f32."""

    # Up to this many (token, expert) pairs per expert the weights are simply streamed once per pair: 4 while an expert is
    # small enough that repeated reads hit L2, 2 above that.
    SMALL_EXPERT_BYTES = 32 << 20

    def __init__(self, w_router, correction, w_gate_up, w_down, top, n_groups, keep_groups, act, renorm=False, rule="grouped_softmax",
                 gated=True, shared=None, group_top=1, weight_scale=1.0):
        if rule not in ("grouped_softmax", "grouped_sigmoid", "top_softmax"):
            raise ValueError(f"unknown routing rule {rule!r}")
        self.group_top, self.weight_scale = int(group_top), float(weight_scale)
        self.w_router, self.correction, self.w_gate_up, self.w_down = w_router, correction, w_gate_up, w_down
        self.top, self.n_groups, self.keep_groups, self.act, self.renorm = top, n_groups, keep_groups, act, renorm
        self.rule, self.gated, self.shared = rule, gated, shared
        self.n_experts = w_gate_up.shape[0]

    def streams_weights(self, n_tok):
        expert_bytes = (self.w_gate_up[0].numel() + self.w_down[0].numel()) * self.w_down.element_size()
        per_expert = 4 if expert_bytes <= self.SMALL_EXPERT_BYTES else 2
        return n_tok * self.top <= per_expert * self.n_experts

    def route(self, h):
        logits = F.linear(h.float(), self.w_router)
        if self.rule == "top_softmax":
            return K.moe_route_top_softmax(logits, self.top)
        if self.rule == "grouped_softmax" and self.group_top == 1 and self.weight_scale == 1.0:
            return K.moe_route(logits, self.correction, self.n_groups, self.keep_groups, self.top, self.renorm)
        fn = K.SCORE_SIGMOID if self.rule == "grouped_sigmoid" else K.SCORE_SOFTMAX
        return K.moe_route_scored(logits, self.correction, self.n_groups, self.keep_groups, self.top, self.renorm, fn, self.group_top,
                                  self.weight_scale)

    def forward(self, h):
        experts, weights = self.route(h)
        if self.streams_weights(h.shape[0]):
            small = K.moe_small if self.gated else K.moe_small_ungated
            out = small(h, self.w_gate_up, self.w_down, experts, weights, self.act)
        else:
            counts, order = K.moe_sort(experts, self.n_experts)
            xs = K.moe_gather(h, order, self.top)
            ys = torch.empty_like(xs)
            spans, at = [], 0
            for e, n in enumerate(counts.tolist()):
                if n:
                    spans.append((e, at, at + n))
                    at += n
            hid = torch.empty(xs.shape[0], self.w_gate_up.shape[1], dtype=xs.dtype, device=xs.device)
            for e, a, b in spans:
                torch.mm(xs[a:b], self.w_gate_up[e].t(), out=hid[a:b])
            if self.gated:                                   # one activation pass over all experts' rows
                hid = K.glu_split(hid, self.act)
            else:
                K.activate_cols(hid, 0, hid.shape[1], self.act)
            for e, a, b in spans:
                torch.mm(hid[a:b], self.w_down[e].t(), out=ys[a:b])
            out = K.moe_combine(ys, order, weights)
        return out if self.shared is None else self.shared.forward_added_to(h, out)
