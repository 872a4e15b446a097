"""ctypes front-end of libmrs_b200_seq.so (include/mrs_b200_seq.h): residual streams, gated linear recurrences,
short causal convolutions, windowed attention over a paged cache, expert routing.  PyTorch supplies memory and the
stream; there is no CPU fallback — a missing library is built on first use (nvcc, sm_100a) or the import fails."""
import ctypes
import os
import subprocess

import torch

from . import ExtensionMissing

_HERE = os.path.dirname(os.path.abspath(__file__))
SEQ_LIB_PATH = os.path.join(_HERE, "libmrs_b200_seq.so")
BF16, F32 = 1, 2
ACT_NONE, ACT_SILU, ACT_GELU_TANH, ACT_SIGMOID, ACT_GELU_ERF, ACT_RELU_SQ = 0, 1, 2, 3, 4, 5
GLU_CAPPED = 100
SCORE_SOFTMAX, SCORE_SIGMOID = 0, 1
QK_NORM_NONE, QK_NORM_HEAD, QK_NORM_WHOLE = 0, 1, 2
DTYPE_CODE = {torch.bfloat16: BF16, torch.float32: F32}
_lib = None


def make_target(directory, product):
    """Build `product` with the Makefile in `directory` when it is missing (a fresh checkout)."""
    if os.path.exists(product):
        return
    try:
        subprocess.check_call(["make", "-s", "-j", str(min(8, os.cpu_count() or 1)), "-C", directory], stdout=subprocess.DEVNULL)
    except (OSError, subprocess.CalledProcessError) as e:
        raise ExtensionMissing(f"{product} is missing and `make -C {directory}` failed: {e}") from e
    if not os.path.exists(product):
        raise ExtensionMissing(f"{product} was not produced by `make -C {directory}`")


def ensure_host_lib():
    from . import kv_index
    make_target(os.path.join(_HERE, "host"), kv_index.HOST_LIB_PATH)
    L = kv_index.host_lib()
    if getattr(L, "_seq_types", None) is None:
        L.mrs_state_slots_new.restype = ctypes.c_void_p
        for f in ("capacity", "num_free", "acquire", "slot_of"):
            getattr(L, f"mrs_state_slots_{f}").restype = ctypes.c_int64
        L._seq_types = True
    return L


class ScanArgs(ctypes.Structure):
    _fields_ = [("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p),
                ("q_ld", ctypes.c_int64), ("k_ld", ctypes.c_int64), ("v_ld", ctypes.c_int64),
                ("dtype", ctypes.c_int), ("act", ctypes.c_int),
                ("heads", ctypes.c_int), ("qk_groups", ctypes.c_int), ("dk", ctypes.c_int), ("dv", ctypes.c_int),
                ("decay_tok", ctypes.c_void_p), ("decay_head", ctypes.c_void_p), ("scale_tok", ctypes.c_void_p),
                ("skip", ctypes.c_void_p), ("state", ctypes.c_void_p),
                ("cu_tok", ctypes.c_void_p), ("past", ctypes.c_void_p), ("slot", ctypes.c_void_p),
                ("n_seq", ctypes.c_int), ("n_tok", ctypes.c_int), ("out", ctypes.c_void_p),
                ("seg_state", ctypes.c_void_p), ("seg_decay", ctypes.c_void_p), ("seg_len", ctypes.c_int), ("n_segs", ctypes.c_int),
                ("decay_vec", ctypes.c_void_p), ("q_scale", ctypes.c_float)]


class GluRule(ctypes.Structure):
    """How a gated feed-forward joins its halves: act(gate) * up, or — act GLU_CAPPED — with g = min(gate, limit) and
    u = clamp(up, -limit, limit): g * sigmoid(slope * g) * (u + shift)."""
    _fields_ = [("act", ctypes.c_int), ("limit", ctypes.c_float), ("slope", ctypes.c_float), ("shift", ctypes.c_float)]

    @classmethod
    def of(cls, act):
        return act if isinstance(act, cls) else cls(int(act), 0.0, 0.0, 0.0)

    @classmethod
    def capped(cls, limit, slope, shift):
        return cls(GLU_CAPPED, float(limit), float(slope), float(shift))


class RmsResidualArgs(ctypes.Structure):
    _fields_ = [("src", ctypes.c_void_p), ("dst", ctypes.c_void_p), ("y", ctypes.c_void_p), ("mult", ctypes.c_float),
                ("hist", ctypes.c_void_p), ("hist_stride", ctypes.c_int64), ("n_hist", ctypes.c_int), ("mix", ctypes.c_void_p),
                ("mixed", ctypes.c_void_p), ("next_w", ctypes.c_void_p), ("eps", ctypes.c_float), ("next_out", ctypes.c_void_p),
                ("dtype", ctypes.c_int), ("n_tok", ctypes.c_int), ("width", ctypes.c_int), ("post_w", ctypes.c_void_p), ("add_vec", ctypes.c_void_p)]


class LatentPrepareArgs(ctypes.Structure):
    _fields_ = [("y", ctypes.c_void_p), ("y_ld", ctypes.c_int64), ("dtype", ctypes.c_int), ("q_col", ctypes.c_int), ("q_rank", ctypes.c_int),
                ("q_norm_w", ctypes.c_void_p), ("q_out", ctypes.c_void_p), ("q_out_ld", ctypes.c_int64),
                ("kv_col", ctypes.c_int), ("kv_rank", ctypes.c_int), ("rot_dim", ctypes.c_int), ("rot_dims", ctypes.c_int),
                ("kv_norm_w", ctypes.c_void_p), ("cos_sin", ctypes.c_void_p), ("eps", ctypes.c_float), ("cache", ctypes.c_void_p),
                ("cache_row", ctypes.c_int64), ("slot_of_tok", ctypes.c_void_p), ("n_tok", ctypes.c_int), ("kv_out", ctypes.c_void_p),
                ("kv_out_ld", ctypes.c_int64)]

class AttnPrepareArgs(ctypes.Structure):
    _fields_ = [("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p),
                ("q_ld", ctypes.c_int64), ("k_ld", ctypes.c_int64), ("v_ld", ctypes.c_int64),
                ("dtype", ctypes.c_int), ("norm_mode", ctypes.c_int),
                ("q_norm_w", ctypes.c_void_p), ("k_norm_w", ctypes.c_void_p), ("eps", ctypes.c_float),
                ("heads", ctypes.c_int), ("kv_heads", ctypes.c_int), ("dk", ctypes.c_int), ("dv", ctypes.c_int),
                ("rot_dims", ctypes.c_int), ("cos_sin", ctypes.c_void_p),
                ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p), ("slot_of_tok", ctypes.c_void_p), ("n_tok", ctypes.c_int)]


class PagedAttentionArgs(ctypes.Structure):
    _fields_ = [("q", ctypes.c_void_p), ("q_ld", ctypes.c_int64), ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p),
                ("dtype", ctypes.c_int), ("heads", ctypes.c_int), ("kv_heads", ctypes.c_int), ("dk", ctypes.c_int), ("dv", ctypes.c_int),
                ("scale", ctypes.c_float), ("window", ctypes.c_int), ("keep_first", ctypes.c_int), ("sink", ctypes.c_void_p),
                ("pages", ctypes.c_void_p), ("pages_ld", ctypes.c_int), ("page_size", ctypes.c_int),
                ("seq_of_tok", ctypes.c_void_p), ("pos_of_tok", ctypes.c_void_p), ("tok_index", ctypes.c_void_p), ("n_tok", ctypes.c_int),
                ("out", ctypes.c_void_p), ("out_ld", ctypes.c_int64), ("out_scale", ctypes.c_float),
                ("k_row", ctypes.c_int64), ("v_row", ctypes.c_int64), ("pool", ctypes.c_int), ("pool_base", ctypes.c_int64),
                ("v_shared", ctypes.c_int), ("out_f32", ctypes.c_int), ("out_head", ctypes.c_int64)]


SCAN_SEGMENT = 256                  # tokens per segment when a long portion is scanned as segments side by side
SCAN_SEGMENT_MIN_TOKENS = 1024      # portions shorter than this run in one pass
SCAN_SCRATCH_BYTES = 1 << 30


def lib():
    global _lib
    if _lib is None:
        make_target(os.path.join(_HERE, "csrc", "seq"), SEQ_LIB_PATH)
        _lib = ctypes.CDLL(SEQ_LIB_PATH)
    return _lib


def _p(t, offset=0):
    """Device address of element `offset` of a tensor (None -> NULL)."""
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr() + offset * t.element_size())


def _st(t):
    return ctypes.c_int64(torch.cuda.current_stream(t.device).cuda_stream)


def _ok(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what} failed: {'bad argument' if rc < 0 else 'cudaError'} {rc}")


_i, _f, _l = ctypes.c_int, ctypes.c_float, ctypes.c_int64


def embed_streams(table, ids, n_streams):
    T, W = ids.numel(), table.shape[1]
    out = torch.empty(T, n_streams, W, dtype=torch.float32, device=table.device)
    _ok(lib().mrs_seq_embed_streams(_p(table), _i(DTYPE_CODE[table.dtype]), _p(ids), _p(out), _i(T), _i(n_streams), _i(W), _st(table)),
        "embed_streams")
    return out


def streams_read_norm(streams, w_in, norm_w, eps, unit_offset, dtype, rows=None):
    T, S, W = streams.shape
    n = T if rows is None else rows.numel()
    out = torch.empty(n, W, dtype=dtype, device=streams.device)
    _ok(lib().mrs_seq_streams_read_norm(_p(streams), _p(w_in), _p(norm_w), _f(eps), _f(unit_offset), _p(rows), _p(out),
                                        _i(DTYPE_CODE[dtype]), _i(n), _i(S), _i(W), _st(streams)), "streams_read_norm")
    return out


def streams_write(streams, w_mix, w_out, y, next_in=None, next_norm_w=None, eps=0.0, unit_offset=0.0):
    """In place on `streams`; returns the next sublayer's normed input when next_norm_w is given."""
    T, S, W = streams.shape
    nxt = torch.empty(T, W, dtype=y.dtype, device=y.device) if next_norm_w is not None else None
    _ok(lib().mrs_seq_streams_write(_p(streams), _p(w_mix), _p(w_out), _p(y), _i(DTYPE_CODE[y.dtype]), _i(T), _i(S), _i(W),
                                    _p(next_in), _p(next_norm_w), _f(eps), _f(unit_offset), _p(nxt), _st(streams)), "streams_write")
    return nxt


def activate_cols(x, col0, cols, act):
    """x[:, col0:col0 + cols] = act(.) in place."""
    _ok(lib().mrs_seq_activate_cols(_p(x, col0), _l(x.stride(0)), _i(DTYPE_CODE[x.dtype]), _i(x.shape[0]), _i(cols), _i(act), _st(x)),
        "activate_cols")


def glu_split(x, act):
    """act: an activation code (act(gate) * up) or a `GluRule`."""
    T, two = x.shape
    out = torch.empty(T, two // 2, dtype=x.dtype, device=x.device)
    rule = GluRule.of(act)
    _ok(lib().mrs_seq_glu_join(_p(x), _p(out), _i(DTYPE_CODE[x.dtype]), _i(T), _i(two // 2), ctypes.byref(rule), _st(x)), "glu_join")
    return out


def bounded_gate(y, col0, cols, bias, lower):
    """f32 [T, cols]: lower + (1 - lower) * sigmoid(y[:, col0:col0 + cols] + bias)."""
    T = y.shape[0]
    out = torch.empty(T, cols, dtype=torch.float32, device=y.device)
    _ok(lib().mrs_seq_bounded_gate(_p(y, col0), _l(y.stride(0)), _i(DTYPE_CODE[y.dtype]), _p(bias), _p(lower), _i(T), _i(cols), _p(out), _st(y)),
        "bounded_gate")
    return out


def power_gate(y, col0, cols, bias, power):
    """f32 [T, cols]: sigmoid(y[:, col0:col0 + cols] + bias) ** power, formed as exp(power * log_sigmoid(.))."""
    T = y.shape[0]
    out = torch.empty(T, cols, dtype=torch.float32, device=y.device)
    _ok(lib().mrs_seq_power_gate(_p(y, col0), _l(y.stride(0)), _i(DTYPE_CODE[y.dtype]), _p(bias), _f(power), _i(T), _i(cols), _p(out), _st(y)),
        "power_gate")
    return out


def gated_group_norm(x, gate, gate_col, weight, groups, eps, gate_act, gate_first, out, out_col=0, out_scale=1.0):
    """x f32 [T, C]; the gate is columns gate_col.. of `gate`; writes columns out_col.. of `out`."""
    T, C = x.shape
    if gate is None:        # no gate: the plain group norm
        _ok(lib().mrs_seq_gated_group_norm(_p(x), _p(None), _l(0), _p(weight), _p(out, out_col), _l(out.stride(0)), _f(out_scale),
                                           _i(DTYPE_CODE[out.dtype]), _i(T), _i(C), _i(groups), _f(eps), _i(ACT_NONE), _i(0), _st(x)),
            "gated_group_norm")
        return
    _ok(lib().mrs_seq_gated_group_norm(_p(x), _p(gate, gate_col), _l(gate.stride(0)), _p(weight), _p(out, out_col), _l(out.stride(0)),
                                       _f(out_scale), _i(DTYPE_CODE[out.dtype]), _i(T), _i(C), _i(groups), _f(eps), _i(gate_act),
                                       _i(int(gate_first)), _st(x)), "gated_group_norm")


def causal_conv(inp, col0, channels, taps, bias, act, conv_state, batch):
    T = inp.shape[0]
    out = torch.empty(T, channels, dtype=inp.dtype, device=inp.device)
    _ok(lib().mrs_seq_causal_conv(_p(inp), _l(inp.stride(0)), _i(col0), _i(DTYPE_CODE[inp.dtype]), _p(taps), _p(bias), _i(channels),
                                  _i(taps.shape[1]), _i(act), _p(conv_state), _p(batch.cu_tok), _p(batch.past), _p(batch.slot),
                                  _p(batch.seq_of_tok), _i(batch.n_seq), _i(T), _p(out), _st(inp)), "causal_conv")
    return out


def ssm_steps(inp, col0, bias, a_log):
    T, H = inp.shape[0], bias.numel()
    step = torch.empty(T, H, dtype=torch.float32, device=inp.device)
    decay = torch.empty_like(step)
    _ok(lib().mrs_seq_ssm_steps(_p(inp), _l(inp.stride(0)), _i(col0), _i(DTYPE_CODE[inp.dtype]), _p(bias), _p(a_log), _i(H), _i(T),
                                _p(step), _p(decay), _st(inp)), "ssm_steps")
    return step, decay


def linear_scan(q, q_col, k, k_col, v, v_col, heads, qk_groups, dk, dv, state, batch, act=ACT_NONE, decay_tok=None, decay_head=None,
                scale_tok=None, skip=None, decay_vec=None, q_scale=1.0):
    """q / k / v are column ranges (starting at *_col) of 2-D activation tensors; returns o f32 [T, heads * dv].
    decay_vec f32 [T, heads * dk]: every state row has its own decay; with k None the key is the decay's complement.
    q_scale: a constant factor on the queries (applied in f32)."""
    T = q.shape[0]
    out = torch.empty(T, heads * dv, dtype=torch.float32, device=q.device)
    a = ScanArgs()
    a.q, a.v = _p(q, q_col).value, _p(v, v_col).value
    a.q_ld, a.v_ld = q.stride(0), v.stride(0)
    if k is not None:
        a.k, a.k_ld = _p(k, k_col).value, k.stride(0)
    a.decay_vec, a.q_scale = _p(decay_vec).value, float(q_scale)
    a.dtype, a.act = DTYPE_CODE[q.dtype], act
    a.heads, a.qk_groups, a.dk, a.dv = heads, qk_groups, dk, dv
    a.decay_tok, a.decay_head = _p(decay_tok).value, _p(decay_head).value
    a.scale_tok, a.skip = _p(scale_tok).value, _p(skip).value
    a.state = state.data_ptr()
    a.cu_tok, a.past, a.slot = batch.cu_tok.data_ptr(), batch.past.data_ptr(), batch.slot.data_ptr()
    a.n_seq, a.n_tok, a.out = batch.n_seq, T, out.data_ptr()
    longest = getattr(batch, "longest", 0)
    if longest >= SCAN_SEGMENT_MIN_TOKENS:
        seg = SCAN_SEGMENT
        while batch.n_seq * -(-longest // seg) * heads * dk * dv * 4 > SCAN_SCRATCH_BYTES:
            seg *= 2
        n_segs = -(-longest // seg)
        if n_segs > 1:
            seg_state = torch.empty(batch.n_seq * n_segs * heads * dk * dv, dtype=torch.float32, device=q.device)
            seg_decay = torch.empty(batch.n_seq * n_segs * heads * (dk if decay_vec is not None else 1), dtype=torch.float32, device=q.device)
            a.seg_state, a.seg_decay, a.seg_len, a.n_segs = seg_state.data_ptr(), seg_decay.data_ptr(), seg, n_segs
    _ok(lib().mrs_seq_linear_scan(ctypes.byref(a), _st(q)), "linear_scan")
    return out


def qk_norm_store(y, q_col, k_col, v_col, q_norm_w, k_norm_w, eps, heads, kv_heads, dk, dv, k_cache, v_cache, slot_of_tok):
    T, ld = y.shape[0], y.stride(0)
    _ok(lib().mrs_seq_qk_norm_store(_p(y, q_col), _l(ld), _p(y, k_col), _l(ld), _p(y, v_col), _l(ld), _i(DTYPE_CODE[y.dtype]),
                                    _p(q_norm_w), _p(k_norm_w), _f(eps), _i(heads), _i(kv_heads), _i(dk), _i(dv), _p(k_cache),
                                    _p(v_cache), _p(slot_of_tok), _i(T), _st(y)), "qk_norm_store")


def window_attention(y, q_col, k_cache, v_cache, heads, kv_heads, dk, dv, scale, window, batch, page_size, out, out_col=0, out_scale=1.0,
                     tok_index=None):
    """Every token of the step (or those listed in tok_index) against the pages of its sequence."""
    n = y.shape[0] if tok_index is None else tok_index.numel()
    _ok(lib().mrs_seq_window_attention(_p(y, q_col), _l(y.stride(0)), _p(k_cache), _p(v_cache), _i(DTYPE_CODE[y.dtype]), _i(heads),
                                       _i(kv_heads), _i(dk), _i(dv), _f(scale), _i(int(window)), _p(batch.pages), _i(batch.pages.shape[1]),
                                       _i(page_size), _p(batch.seq_of_tok), _p(batch.pos_of_tok), _p(tok_index), _i(n), _p(out, out_col),
                                       _l(out.stride(0)), _f(out_scale), _st(y)), "window_attention")


def scale_rows(x, row0, rows, col0, cols, scale):
    _ok(lib().mrs_seq_scale_rows(_p(x, row0 * x.stride(0) + col0), _l(x.stride(0)), _i(DTYPE_CODE[x.dtype]), _i(rows), _i(cols), _f(scale),
                                 _st(x)), "scale_rows")


def fresh_prompt_attention(y, row0, rows, q_col, k_col, v_col, heads, kv_heads, d, scale, window, out, out_col):
    """Causal (windowed) attention of one sequence's first `rows` tokens over its own fresh q / k / v, through the
    package's prompt-attention kernels (tcgen05 for head size 128 without a window, mma.sync otherwise; libmrs_b200.so,
    built on first use).  q / k / v are column ranges of `y`; writes heads * d columns of `out` from out_col."""
    from . import LIB_PATH, lib as main_lib
    make_target(os.path.join(_HERE, "csrc"), LIB_PATH)
    ld, at = y.stride(0), row0 * y.stride(0)
    rc = main_lib().mrs_prefill_attention(_p(y, at + q_col), _p(y, at + k_col), _p(y, at + v_col), _p(out, row0 * out.stride(0) + out_col),
                                          ctypes.c_void_p(0), _i(0), _i(rows), _i(rows), _i(heads), _i(kv_heads), _i(d), _l(ld), _l(ld),
                                          _l(out.stride(0)), _f(scale), _i(1), _i(window - 1 if window > 0 else -1), _f(0.0),
                                          ctypes.c_uint32(1), ctypes.c_void_p(torch.cuda.current_stream(y.device).cuda_stream))
    _ok(rc, "mrs_prefill_attention")


def moe_route(logits, correction, n_groups, keep_groups, top, renorm=False):
    T, E = logits.shape
    experts = torch.empty(T, top, dtype=torch.int32, device=logits.device)
    weights = torch.empty(T, top, dtype=torch.float32, device=logits.device)
    _ok(lib().mrs_seq_moe_route(_p(logits), _p(correction), _i(T), _i(E), _i(n_groups), _i(keep_groups), _i(top), _i(int(renorm)),
                                _p(experts), _p(weights), _st(logits)), "moe_route")
    return experts, weights


def moe_route_scored(logits, correction, n_groups, keep_groups, top, renorm=False, score_fn=SCORE_SOFTMAX, group_top=1, weight_scale=1.0):
    """`moe_route` with its choices open: softmax or sigmoid scores, a group scored by the sum of its group_top largest
    choices, weights times weight_scale."""
    T, E = logits.shape
    experts = torch.empty(T, top, dtype=torch.int32, device=logits.device)
    weights = torch.empty(T, top, dtype=torch.float32, device=logits.device)
    _ok(lib().mrs_seq_moe_route_scored(_p(logits), _p(correction), _i(T), _i(E), _i(n_groups), _i(keep_groups), _i(top), _i(int(renorm)),
                                       _i(score_fn), _i(group_top), _f(weight_scale), _p(experts), _p(weights), _st(logits)), "moe_route_scored")
    return experts, weights


def moe_small(x, gate_up, down, experts, weights, act):
    """Expert feed-forward by weight streaming (few tokens): gate_up [E, 2ff, W], down [E, W, ff]; act: a code or a `GluRule`."""
    T, W = x.shape
    top, ff = experts.shape[1], down.shape[2]
    code = _i(DTYPE_CODE[x.dtype])
    hidden = torch.empty(T * top, ff, dtype=x.dtype, device=x.device)
    out = torch.empty(T, W, dtype=x.dtype, device=x.device)
    rule = GluRule.of(act)
    _ok(lib().mrs_seq_moe_gate_up_rule(_p(x), _p(gate_up), code, _p(experts), _i(T), _i(top), _i(W), _i(ff), ctypes.byref(rule), _p(hidden),
                                       _st(x)), "moe_gate_up")
    _ok(lib().mrs_seq_moe_down(_p(hidden), _p(down), code, _p(experts), _p(weights), _i(T), _i(top), _i(W), _i(ff), _p(out), _st(x)),
        "moe_down")
    return out


def moe_sort(experts, n_experts):
    n = experts.numel()
    counts = torch.empty(n_experts, dtype=torch.int32, device=experts.device)
    order = torch.empty(n, dtype=torch.int32, device=experts.device)
    _ok(lib().mrs_seq_moe_sort(_p(experts), _i(n), _i(n_experts), _p(counts), _p(order), _st(experts)), "moe_sort")
    return counts, order


def moe_gather(x, order, top):
    n, W = order.numel(), x.shape[1]
    out = torch.empty(n, W, dtype=x.dtype, device=x.device)
    _ok(lib().mrs_seq_moe_gather(_p(x), _i(DTYPE_CODE[x.dtype]), _p(order), _i(n), _i(top), _i(W), _p(out), _st(x)), "moe_gather")
    return out


def moe_combine(sorted_y, order, weights):
    T, top = weights.shape
    W = sorted_y.shape[1]
    inverse = torch.empty(T * top, dtype=torch.int32, device=sorted_y.device)
    out = torch.empty(T, W, dtype=sorted_y.dtype, device=sorted_y.device)
    _ok(lib().mrs_seq_moe_combine(_p(sorted_y), _i(DTYPE_CODE[sorted_y.dtype]), _p(order), _p(weights), _i(T), _i(top), _i(W),
                                  _p(inverse), _p(out), _st(sorted_y)), "moe_combine")
    return out


# ---- single residual with Dynamic Tanh norms ------------------------------------------------------------
def tanh_norm_rows(x, norm, dtype, rows=None):
    """dyt(x[rows]) for the f32 residual x [T, W]; norm = (alpha, weight, bias) f32 on the device."""
    T, W = x.shape
    n = T if rows is None else rows.numel()
    out = torch.empty(n, W, dtype=dtype, device=x.device)
    _ok(lib().mrs_seq_tanh_norm_rows(_p(x), _p(rows), _p(norm[0]), _p(norm[1]), _p(norm[2]), _p(out), _i(DTYPE_CODE[dtype]), _i(n), _i(W),
                                     _st(x)), "tanh_norm_rows")
    return out


def residual_tanh_norm(x, y=None, post=None, extra=None, nxt=None, dtype=None):
    """In place on the f32 residual: x += dyt_post(y); x += extra; returns dyt_next(x) when nxt is given (each part optional)."""
    T, W = x.shape
    dtype = y.dtype if y is not None else dtype
    out = torch.empty(T, W, dtype=dtype, device=x.device) if nxt is not None else None
    post, nxt = post or (None, None, None), nxt or (None, None, None)
    _ok(lib().mrs_seq_residual_tanh_norm(_p(x), _p(y), _i(DTYPE_CODE[dtype]), _p(post[0]), _p(post[1]), _p(post[2]), _p(extra), _p(nxt[0]),
                                         _p(nxt[1]), _p(nxt[2]), _p(out), _i(T), _i(W), _st(x)), "residual_tanh_norm")
    return out


# ---- attention: general preparation, rotation table, sink / kept-first window ---------------------------
def rotation_table(pos_of_tok, freq, mag):
    """f32 [T, half, 2]: mag * (cos, sin)(pos * freq), angles in double.  freq: f64 on the device."""
    T, half = pos_of_tok.numel(), freq.numel()
    out = torch.empty(T, half, 2, dtype=torch.float32, device=freq.device)
    _ok(lib().mrs_seq_rotation_table(_p(pos_of_tok), _p(freq), _i(T), _i(half), _f(mag), _p(out), _st(freq)), "rotation_table")
    return out


def attention_prepare(y, q_col, k_col, v_col, norm_mode, q_norm_w, k_norm_w, eps, heads, kv_heads, dk, dv, k_cache, v_cache, slot_of_tok,
                      cos_sin=None, rot_dims=0):
    """q | k | v are column ranges of y.  v_col None: the values are the keys as projected."""
    a = AttnPrepareArgs()
    ld = y.stride(0)
    a.q, a.k, a.q_ld, a.k_ld = _p(y, q_col).value, _p(y, k_col).value, ld, ld
    if v_col is not None:
        a.v, a.v_ld = _p(y, v_col).value, ld
    a.dtype, a.norm_mode = DTYPE_CODE[y.dtype], norm_mode
    a.q_norm_w, a.k_norm_w, a.eps = _p(q_norm_w).value, _p(k_norm_w).value, eps
    a.heads, a.kv_heads, a.dk, a.dv = heads, kv_heads, dk, dv
    a.rot_dims, a.cos_sin = rot_dims, _p(cos_sin).value
    a.k_cache, a.v_cache, a.slot_of_tok, a.n_tok = k_cache.data_ptr(), v_cache.data_ptr(), slot_of_tok.data_ptr(), y.shape[0]
    _ok(lib().mrs_seq_attention_prepare(ctypes.byref(a), _st(y)), "attention_prepare")


def paged_attention(y, q_col, k_cache, v_cache, heads, kv_heads, dk, dv, scale, window, keep_first, sink, batch, page_size, out, out_col=0,
                    out_scale=1.0, tok_index=None, k_row=0, v_row=0, pool=0, pool_base=0, v_shared=False, v_col=0, out_head=0):
    """Every token of the step (or those listed in tok_index) against the pages of its sequence: position i sees j <= i
    with i - j < window (0: all) or j < keep_first; sink [heads] f32 or None.  k_row / v_row: elements between the cache
    rows of neighbouring slots (0: kv_heads * dk / kv_heads * dv).  pool > 0: besides the window, one averaged entry per
    block of `pool` positions wholly before it, read from cache rows pool_base.. (`pool_blocks`).  v_shared: every head
    reads value columns [v_col, v_col + dv) of a row — dv is then several (or all) value heads side by side, and out_head the
    distance between the heads of an output row.  An f32 `out` is written as f32 whatever the activation type."""
    a = PagedAttentionArgs()
    a.k_row, a.v_row = int(k_row), int(v_row)
    a.pool, a.pool_base, a.v_shared = int(pool), int(pool_base), int(bool(v_shared))
    a.out_f32 = int(out.dtype == torch.float32 and y.dtype != torch.float32)
    a.q, a.q_ld, a.k_cache, a.v_cache = _p(y, q_col).value, y.stride(0), k_cache.data_ptr(), _p(v_cache, int(v_col)).value
    a.out_head = int(out_head)
    a.dtype, a.heads, a.kv_heads, a.dk, a.dv = DTYPE_CODE[y.dtype], heads, kv_heads, dk, dv
    a.scale, a.window, a.keep_first, a.sink = scale, int(window), int(keep_first), _p(sink).value
    a.pages, a.pages_ld, a.page_size = batch.pages.data_ptr(), batch.pages.shape[1], page_size
    a.seq_of_tok, a.pos_of_tok, a.tok_index = batch.seq_of_tok.data_ptr(), batch.pos_of_tok.data_ptr(), _p(tok_index).value
    a.n_tok = y.shape[0] if tok_index is None else tok_index.numel()
    a.out, a.out_ld, a.out_scale = _p(out, out_col).value, out.stride(0), out_scale
    _ok(lib().mrs_seq_paged_attention(ctypes.byref(a), _st(y)), "paged_attention")


def dense_prompt_attention(q, q_col, k, v, batch, heads, kv_heads, d, scale, window, sink, out, out_col=0):
    """The tensor-core prompt kernel over keys and values that are DENSE rows of the step (k, v [T, kv_heads * d], row t = the
    step's token t) instead of pages: for steps whose sequences all start in this step with a long portion.  The kernel's page
    table becomes one row per sequence listing its tokens' rows (page size 1); built once per step."""
    if len(batch.long) != batch.n_seq or any(past for _, _, past, _ in batch.long):
        raise ValueError("dense keys cover the step's own tokens only: every sequence must start in this step with a long portion")
    plan = batch.__dict__.get("_dense_rows")
    if plan is None:
        rows = batch.long_rows.view(-1, 4)
        table = (rows[:, 0:1] + torch.arange(batch.longest, dtype=torch.int32, device=rows.device)[None, :]).contiguous()
        portions = rows.clone()
        portions[:, 3] = torch.arange(rows.shape[0], dtype=torch.int32, device=rows.device)
        plan = batch.__dict__["_dense_rows"] = (table, portions.contiguous())
    table, portions = plan
    _ok(lib().mrs_seq_prompt_attention_pooled(_p(q, q_col), _l(q.stride(0)), _p(k), _p(v), _p(out, out_col), _l(out.stride(0)), _p(portions),
                                              _i(len(batch.long)), _i(batch.longest), _p(table), _i(table.shape[1]), _i(1), _i(heads), _i(kv_heads),
                                              _i(d), _f(scale), _i(int(window)), _i(0), _p(sink), _i(0), _l(0), _i(0), _st(q)), "dense_prompt_attention")


def pool_rows(n_token_slots, page_size, pool):
    """Cache rows that the averaged blocks of a pool of n_token_slots token rows need (per page: as many as blocks can start in one)."""
    return (n_token_slots // page_size) * (-(-page_size // pool))


def pool_blocks(k_cache, v_cache, k_cols, v_cols, pool, pool_base, batch, page_size):
    """For every token of the step that ends a block of `pool` positions: the block's mean key / value row -> its cache row."""
    _ok(lib().mrs_seq_pool_blocks(_p(k_cache), _p(v_cache), _i(DTYPE_CODE[k_cache.dtype]), _l(k_cols), _l(v_cols), _i(k_cols), _i(v_cols),
                                  _i(pool), _l(pool_base), _p(batch.pages), _i(batch.pages.shape[1]), _i(page_size), _p(batch.seq_of_tok),
                                  _p(batch.pos_of_tok), _i(batch.n_tok), _st(k_cache)), "pool_blocks")


def mix_heads(a, mix, heads, kv_heads, dv, out, gate=None, gate_col=0, gate_act=ACT_NONE):
    """out[t, h] = act(gate[t, h]) * sum_g mix[h, g] * a[t, g, value head of h]; a f32 [T, heads * kv_heads * dv]."""
    _ok(lib().mrs_seq_mix_heads(_p(a), _p(mix), _p(gate, gate_col) if gate is not None else _p(None), _l(gate.stride(0) if gate is not None else 0),
                                _i(gate_act), _p(out), _l(out.stride(0)), _i(DTYPE_CODE[out.dtype]), _i(heads), _i(kv_heads), _i(dv),
                                _i(out.shape[0]), _st(out)), "mix_heads")


def gate_cols(x, gate, gate_col, cols, group, act):
    """x[:, c] *= act(gate[:, gate_col + c // group]) in place for c < cols."""
    _ok(lib().mrs_seq_gate_cols(_p(x), _l(x.stride(0)), _p(gate, gate_col), _l(gate.stride(0)), _i(DTYPE_CODE[x.dtype]), _i(cols), _i(group),
                                _i(act), _i(x.shape[0]), _st(x)), "gate_cols")


def prompt_attention(y, q_col, k_cache, v_cache, batch, page_size, heads, kv_heads, d, scale, window, keep_first, sink, out, out_col=0, pool=0,
                     pool_base=0, every_value_head=False):
    """The long portions of the step (batch.long: fresh or continued) on tensor cores: queries from their rows of y, keys
    and values from the pages (bf16, head size 64 or 128).  pool / pool_base: averaged blocks before the window, as for
    `paged_attention`.  every_value_head: `out` is f32 [T, heads * kv_heads * d], every head's weights on every value head."""
    _ok(lib().mrs_seq_prompt_attention_pooled(_p(y, q_col), _l(y.stride(0)), _p(k_cache), _p(v_cache), _p(out, out_col), _l(out.stride(0)),
                                              _p(batch.long_rows), _i(len(batch.long)), _i(max(n for _, n, _, _ in batch.long)), _p(batch.pages),
                                              _i(batch.pages.shape[1]), _i(page_size), _i(heads), _i(kv_heads), _i(d), _f(scale), _i(int(window)),
                                              _i(int(keep_first)), _p(sink), _i(int(pool)), _l(int(pool_base)), _i(int(bool(every_value_head))),
                                              _st(y)), "prompt_attention")


# ---- stabilised matrix memory ---------------------------------------------------------------------------
def mlstm_gates(raw, heads, cap, m_state, batch):
    """raw f32 [T, 2 * heads] (input gates | forget gates, biases added) -> keep, take, m f32 [T, heads]; advances m_state."""
    T = raw.shape[0]
    keep = torch.empty(T, heads, dtype=torch.float32, device=raw.device)
    take, m_tok = torch.empty_like(keep), torch.empty_like(keep)
    _ok(lib().mrs_seq_mlstm_gates(_p(raw), _p(raw, heads), _l(raw.stride(0)), _f(cap), _i(heads), _p(m_state), _p(batch.cu_tok),
                                  _p(batch.past), _p(batch.slot), _i(batch.n_seq), _i(T), _p(keep), _p(take), _p(m_tok), _st(raw)),
        "mlstm_gates")
    return keep, take, m_tok


def append_ones(y, v_col, heads, dv, dvp):
    out = torch.empty(y.shape[0], heads * dvp, dtype=y.dtype, device=y.device)
    _ok(lib().mrs_seq_append_ones(_p(y, v_col), _l(y.stride(0)), _i(DTYPE_CODE[y.dtype]), _i(heads), _i(dv), _i(dvp), _i(y.shape[0]), _p(out),
                                  _st(y)), "append_ones")
    return out


def mlstm_out_norm(o, dvp, m_tok, q_scale, gate, gate_col, weight, eps, heads, dv, dtype):
    T = o.shape[0]
    out = torch.empty(T, heads * dv, dtype=dtype, device=o.device)
    _ok(lib().mrs_seq_mlstm_out_norm(_p(o), _i(dvp), _p(m_tok), _f(q_scale), _p(gate, gate_col), _l(gate.stride(0)), _p(weight), _f(eps),
                                     _i(heads), _i(dv), _p(out), _l(out.stride(0)), _i(DTYPE_CODE[dtype]), _i(T), _st(o)), "mlstm_out_norm")
    return out


# ---- experts: plain top-k rule, experts without a gate -----------------------------------------------------
def moe_route_top_softmax(logits, top):
    T, E = logits.shape
    experts = torch.empty(T, top, dtype=torch.int32, device=logits.device)
    weights = torch.empty(T, top, dtype=torch.float32, device=logits.device)
    _ok(lib().mrs_seq_moe_route_top_softmax(_p(logits), _i(T), _i(E), _i(top), _p(experts), _p(weights), _st(logits)), "moe_route_top_softmax")
    return experts, weights


def moe_small_ungated(x, up, down, experts, weights, act):
    """Expert feed-forward without a gate by weight streaming (few tokens): up [E, ff, W], down [E, W, ff]."""
    T, W = x.shape
    top, ff = experts.shape[1], down.shape[2]
    code = _i(DTYPE_CODE[x.dtype])
    hidden = torch.empty(T * top, ff, dtype=x.dtype, device=x.device)
    out = torch.empty(T, W, dtype=x.dtype, device=x.device)
    _ok(lib().mrs_seq_moe_up(_p(x), _p(up), code, _p(experts), _i(T), _i(top), _i(W), _i(ff), _i(act), _p(hidden), _st(x)), "moe_up")
    _ok(lib().mrs_seq_moe_down(_p(hidden), _p(down), code, _p(experts), _p(weights), _i(T), _i(top), _i(W), _i(ff), _p(out), _st(x)),
        "moe_down")
    return out


# ---- single residual with RMS norms, a multiplier and a depth-weighted average ---------------------------------
def embed_scaled(table, ids, scale, out):
    """out f32 [T, W] = table[ids] * scale."""
    T, W = ids.numel(), table.shape[1]
    _ok(lib().mrs_seq_embed_scaled(_p(table), _i(DTYPE_CODE[table.dtype]), _p(ids), _f(scale), _p(out), _i(T), _i(W), _st(table)), "embed_scaled")
    return out


def embed_pair(table, pairs, ids, scale, buckets, mul_prev, mul_cur, prev_state, batch, out):
    """out f32 [T, W] = table[ids] * scale + pairs[hash of (previous token, token)]; the table's last row for a sequence's first
    token; prev_state int32 [slots] carries every request's last token from step to step."""
    T, W = ids.numel(), table.shape[1]
    _ok(lib().mrs_seq_embed_pair(_p(table), _p(pairs), _i(DTYPE_CODE[table.dtype]), _p(ids), _f(scale), _l(buckets), _l(mul_prev), _l(mul_cur),
                                 _p(prev_state), _p(batch.cu_tok), _p(batch.past), _p(batch.slot), _p(batch.seq_of_tok), _p(out), _i(T), _i(W),
                                 _st(table)), "embed_pair")
    return out


def rms_residual(src, y=None, mult=1.0, dst=None, hist=None, n_hist=0, mix=None, mixed=None, next_w=None, eps=0.0, dtype=None, post_w=None,
                 add_vec=None):
    """One pass over an f32 residual [T, W]: v = src + mult * y (y first RMS-normed with post_w when given) + add_vec [W] -> dst;
    v = sum_j mix[j] * hist[j] (hist f32 [>= n_hist, T, W], dst may be one of its entries) -> mixed; returns rms_norm(v) * next_w
    in the activation type when next_w is given."""
    T, W = src.shape
    dtype = y.dtype if y is not None else dtype
    out = torch.empty(T, W, dtype=dtype, device=src.device) if next_w is not None else None
    a = RmsResidualArgs()
    a.src, a.dst, a.y, a.mult = _p(src).value, _p(dst).value, _p(y).value, float(mult)
    if hist is not None:
        a.hist, a.hist_stride, a.n_hist, a.mix = _p(hist).value, hist.stride(0), int(n_hist), _p(mix).value
    a.mixed, a.next_w, a.eps, a.next_out = _p(mixed).value, _p(next_w).value, float(eps), _p(out).value
    a.dtype, a.n_tok, a.width = DTYPE_CODE[dtype], T, W
    a.post_w, a.add_vec = _p(post_w).value, _p(add_vec).value
    _ok(lib().mrs_seq_rms_residual(ctypes.byref(a), _st(src)), "rms_residual")
    return out


# ---- attention through a shared latent -----------------------------------------------------------------------
def latent_prepare(y, q_col, q_rank, q_norm_w, q_out, kv_col, kv_rank, rot_dim, rot_dims, kv_norm_w, cos_sin, eps, cache, slot_of_tok, kv_out=None):
    """From the columns of y: q_out = rms_norm(query latent) * w; cache[slot] = rms_norm(key/value latent) * w | the shared key
    part turned in neighbouring pairs.  kv_rank 0: only the query part.  kv_out [T, >= kv_rank]: the normed latent also as dense rows."""
    a = LatentPrepareArgs()
    a.y, a.y_ld, a.dtype = _p(y).value, y.stride(0), DTYPE_CODE[y.dtype]
    a.q_col, a.q_rank, a.q_norm_w = int(q_col), int(q_rank), _p(q_norm_w).value
    if q_out is not None:
        a.q_out, a.q_out_ld = _p(q_out).value, q_out.stride(0)
    a.kv_col, a.kv_rank, a.rot_dim, a.rot_dims = int(kv_col), int(kv_rank), int(rot_dim), int(rot_dims)
    a.kv_norm_w, a.cos_sin, a.eps = _p(kv_norm_w).value, _p(cos_sin).value, float(eps)
    if kv_rank:
        a.cache, a.cache_row, a.slot_of_tok = _p(cache).value, cache.stride(0), _p(slot_of_tok).value
    a.n_tok = y.shape[0]
    if kv_out is not None:
        a.kv_out, a.kv_out_ld = _p(kv_out).value, kv_out.stride(0)
    _ok(lib().mrs_seq_latent_prepare(ctypes.byref(a), _st(y)), "latent_prepare")


def rotate_pairs(src, src_col, src_head, dst, dst_col, dst_head, heads, dims, rot_dims, cos_sin):
    """dst[t, dst_col + h * dst_head + d] = src[t, src_col + h * src_head + d], d < dims, the first rot_dims turned in
    neighbouring pairs by cos_sin [T, rot_dims / 2, 2]."""
    _ok(lib().mrs_seq_rotate_pairs(_p(src, src_col), _l(src.stride(0)), _l(src_head), _p(dst, dst_col), _l(dst.stride(0)), _l(dst_head),
                                   _i(DTYPE_CODE[src.dtype]), _i(heads), _i(dims), _i(rot_dims), _p(cos_sin), _i(src.shape[0]), _st(src)),
        "rotate_pairs")


def latent_attention_fits(kv_rank, rot_dim):
    """True when the tensor-core latent kernel takes these sizes (bf16 only)."""
    return bool(lib().mrs_seq_latent_attention_fits(_i(kv_rank), _i(rot_dim)))


def latent_prompt_attention(qa, latent, heads, kv_rank, rot_dim, scale, window, batch, page_size, out):
    """Absorbed latent attention of every sequence of the step on tensor cores: prompt portions of any length and single
    decoded tokens alike (a token's heads are rows of one tile; the window's latents are fetched once for all of them)."""
    _ok(lib().mrs_seq_latent_attention(_p(qa), _l(qa.stride(0)), _p(latent), _l(latent.stride(0)), _p(out), _l(out.stride(0)),
                                       _p(None), _p(batch.cu_tok), _p(batch.past), _i(batch.n_seq), _i(batch.longest), _p(batch.pages),
                                       _i(batch.pages.shape[1]), _i(page_size), _i(heads), _i(kv_rank), _i(rot_dim), _f(scale), _i(int(window)),
                                       _st(qa)), "latent_attention")


def latent_attention(qa, latent, heads, kv_rank, rot_dim, scale, window, batch, page_size, out, tok_index=None):
    """Absorbed latent attention of every token of the step: qa [T, heads * (kv_rank + rot_dim)] against the cached latent
    rows [slots, >= kv_rank + rot_dim] as one key/value head (values = the rows' first kv_rank columns); out [T, heads * kv_rank]."""
    paged_attention(qa, 0, latent, latent, heads, 1, kv_rank + rot_dim, kv_rank, scale, window, 0, None, batch, page_size, out,
                    tok_index=tok_index, k_row=latent.stride(0), v_row=latent.stride(0))
