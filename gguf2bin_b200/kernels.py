"""Python bindings of the CUDA kernels (ctypes over the C launchers of ``csrc/``).

Every function takes CUDA tensors, launches on the current torch stream and returns
nothing or its output tensor.  There is no CPU path: a tensor that is not on a CUDA
device raises ``KernelError``, and a missing or unbuildable extension raises
``KernelBuildError`` at the first call.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_ulonglong, c_void_p
from typing import Optional

import torch

from .csrc.build import KernelBuildError, KernelError, load_unit

__all__ = ["KernelError", "KernelBuildError", "embed_rows", "rmsnorm", "qknorm_rope_cache",
           "rope_table", "cache_write", "swiglu", "advance_positions", "gemm_simt", "linear", "attn_generic",
           "attention", "sample_rows", "sample_filtered", "recent_set", "seed_slots", "embed_pair_norm",
           "canon_conv", "norm_canon_single", "latent_keep", "head_product", "head_gate", "gated_add", "xielu",
           "proj_norm_rope_cache", "rotate_heads", "short_conv", "state_scan", "head_norm_gate", "gate_mul",
           "norm_add", "norm_shift", "scan_gates_step", "scan_gates_max", "state_readout", "pool_update", "moe_route", "moe_plan", "moe_gemm", "moe_gemv", "moe_gather", "moe_gemm_tc", "moe_combine", "moe_combine_norm_add", "moe_tile_rows", "tanh_norm", "scaled_join", "relu2", "selective_scan", "diff_combine"]

F32, BF16 = 0, 1
EPI_STORE_F32, EPI_STORE_BF16, EPI_ACCUM_F32 = 0, 1, 2


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dtype}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernel called with a tensor that is not on a CUDA device "
                          "(there is no CPU path)")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """Handle of the current stream of the current device (the direct bindings when this
    torch has them: a launch costs microseconds on the host, and this is asked once per launch)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, dtype: torch.dtype, what: str) -> None:
    if t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


_fn_cache: dict = {}
_bf16 = None              # the bfloat16 bindings (they import this module, so they are bound at first use)


def _bf16_mod():
    global _bf16
    if _bf16 is None:
        from . import kernels_bf16 as m
        _bf16 = m
    return _bf16


def _fn(unit: str, name: str, argtypes, defines=()):
    key = (unit, name, tuple(defines))
    f = _fn_cache.get(key)
    if f is None:
        lib = load_unit(unit, defines)
        f = getattr(lib, name)
        f.argtypes = argtypes
        f.restype = c_int
        f._lib = lib
        _fn_cache[key] = f
    return f


_launches = 0
_scratch: dict = {}       # small persistent device buffers of the bindings, by (device, use)
_scratch_outgrown: list = []     # buffers that were replaced by larger ones: a captured graph may still use them


def _scratch_buffer(key, n: int, dtype) -> torch.Tensor:
    """The persistent buffer of that use with at least ``n`` elements.  A buffer that is
    outgrown is kept, not freed: launches captured in a CUDA graph go on writing to it."""
    buf = _scratch.get(key)
    if buf is None or buf.numel() < n or buf.dtype != dtype:
        if buf is not None:
            _scratch_outgrown.append(buf)
        buf = _scratch[key] = torch.empty(n, dtype=dtype, device=key[0])
    return buf


def launch_count() -> int:
    """How many kernels the launchers called so far in this process have launched."""
    return _launches


def count_launches(n: int) -> None:
    """A launcher that starts more than one kernel per call adds the others here."""
    global _launches
    _launches += n


def _call(f, *args) -> None:
    global _launches
    _launches += 1
    rc = f(*args)
    if rc != 0:
        raise KernelError(f._lib.g2b_last_error().decode("utf-8", "replace"))


# ---------------------------------------------------------------------------
# elementwise.cu
# ---------------------------------------------------------------------------
def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] widened to float32, times ``scale``.  ids int32 [T], out float32 [T, H]."""
    _need(ids, torch.int32, "ids")
    _need(out, torch.float32, "out")
    V, H = table.shape
    f = _fn("elementwise.cu", "g2b_embed_rows",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _call(f, _ptr(table), _code(table.dtype), _ptr(ids), _ptr(out), out.shape[0], H, V, float(scale), _stream())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = (w * x[row_r]) / sqrt(mean(x[row_r]^2) + eps); x, w float32 (w None: all
    ones); statistics in float32.  ``rows`` (int32) gathers rows of x; out has one row per gathered row."""
    _need(x, torch.float32, "x")
    if w is not None:                      # None: no per-channel weight
        _need(w, torch.float32, "norm weight")
    if rows is not None:
        _need(rows, torch.int32, "rows")
    n_rows, H = out.shape
    f = _fn("elementwise.cu", "g2b_rmsnorm",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_int, c_void_p])
    _call(f, _ptr(x), _ptr(w), _ptr(rows), n_rows, H, eps, _ptr(out), _code(out.dtype), _stream())


def tanh_norm(x: torch.Tensor, alpha: torch.Tensor, w: torch.Tensor, b: torch.Tensor, out: torch.Tensor,
              rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = tanh(alpha * x[row_r]) * w + b: a norm that takes no statistics of the row.  x, w, b
    float32, ``alpha`` float32 with one element (read on the device); ``rows`` (int32) gathers rows."""
    _need(x, torch.float32, "x")
    for t, what in ((alpha, "alpha"), (w, "norm weight"), (b, "norm bias")):
        _need(t, torch.float32, what)
    if rows is not None:
        _need(rows, torch.int32, "rows")
    if not out.is_contiguous():
        raise KernelError("tanh_norm: out must be contiguous")
    n_rows, H = out.shape
    f = _fn("elementwise.cu", "g2b_tanh_norm",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p])
    _call(f, _ptr(x), _ptr(alpha), _ptr(w), _ptr(b), _ptr(rows), n_rows, H, _ptr(out), _code(out.dtype), _stream())


def scaled_join(x32, y1, s1, y2=None, s2=None, norm=None, normed_out=None) -> None:
    """x += y1 * s1 (+ y2 * s2): sublayer results [T, H] join the stream, each times one learned number
    per channel ([H]); everything float32.  ``norm`` = (alpha, w, b) with ``normed_out`` [T, H] (compute type):
    the new rows also leave as tanh(alpha x) * w + b, the next layer's norm, in the same pass."""
    for t, what in ((x32, "stream"), (y1, "result"), (s1, "scale")):
        _need(t, torch.float32, what)
    if y2 is not None:
        _need(y2, torch.float32, "second result")
        _need(s2, torch.float32, "second scale")
    alpha = w = b = None
    if norm is not None:
        alpha, w, b = norm
        for t, what in ((alpha, "alpha"), (w, "norm weight"), (b, "norm bias")):
            _need(t, torch.float32, what)
        if normed_out is None or not normed_out.is_contiguous() or tuple(normed_out.shape) != tuple(x32.shape):
            raise KernelError("scaled_join: the normed rows need a contiguous output of the stream's shape")
    f = _fn("elementwise.cu", "g2b_scaled_join", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                                   c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _call(f, _ptr(x32), _ptr(y1), _ptr(s1), _ptr(y2), _ptr(s2) if y2 is not None else None, x32.shape[0], x32.shape[1],
          _ptr(alpha), _ptr(w), _ptr(b), _ptr(normed_out) if norm is not None else None,
          _code(normed_out.dtype) if norm is not None else F32, _stream())


def relu2(z, out) -> None:
    """out = max(z, 0)^2; z [T, F] a view with any row stride, out [T, F] contiguous, one dtype."""
    if z.stride(1) != 1 or out.dtype != z.dtype or not out.is_contiguous():
        raise KernelError("relu2: dense rows of one dtype")
    f = _fn("elementwise.cu", "g2b_relu2", [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _call(f, _ptr(z), z.stride(0), _code(z.dtype), z.shape[0], z.shape[1], _ptr(out), _stream())


def rope_table(tok_pos: torch.Tensor, inv_freq: torch.Tensor, table: torch.Tensor, mult: float = 1.0) -> None:
    """table[t, j] = (cos, sin)(tok_pos[t] * inv_freq[j]) * mult in float32; table [T, half, 2]."""
    _need(tok_pos, torch.int32, "tok_pos")
    _need(inv_freq, torch.float32, "inv_freq")
    _need(table, torch.float32, "table")
    f = _fn("elementwise.cu", "g2b_rope_table", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p])
    _call(f, _ptr(tok_pos), _ptr(inv_freq), _ptr(table), table.shape[0], inv_freq.shape[0], float(mult), _stream())


def qknorm_rope_cache(qkv, n_heads, n_kv_heads, head_dim, q_w, k_w, eps, rope, rotary_dim,
                      tok_pos, tok_seq, page_table, cache_pages, page_size, q_out,
                      k_out=None, v_out=None) -> None:
    """Per-head RMSNorm of the q and k heads (when q_w / k_w are given), half-split
    rotation by the angles of ``rope`` (a table from ``rope_table`` for this step's
    tokens; None: no rotation), q to ``q_out``; k and v to the layer's cache pages, or to
    ``k_out`` / ``v_out`` when those are given."""
    T = qkv.shape[0]
    f = _fn("elementwise.cu", "g2b_qknorm_rope_cache",
            [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p,
             c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
             c_void_p, c_void_p])
    P = page_table.shape[1] if page_table is not None else 0
    for t in (q_out, k_out, v_out, cache_pages):
        if t is not None and t.dtype != qkv.dtype:
            raise KernelError("qknorm_rope_cache: outputs and cache must have the input's dtype")
    _call(f, _ptr(qkv), _code(qkv.dtype), T, n_heads, n_kv_heads, head_dim, _ptr(q_w), _ptr(k_w),
          eps, _ptr(rope), rotary_dim, _ptr(tok_pos), _ptr(tok_seq), _ptr(page_table), P,
          _ptr(cache_pages), page_size, _ptr(q_out), _ptr(k_out), _ptr(v_out), _stream())


def cache_write(k, v, n_kv_heads, head_dim, tok_pos, tok_seq, page_table, cache_pages,
                page_size) -> None:
    """k, v [T, n_kv_heads*head_dim] into the layer's cache pages at each token's position."""
    f = _fn("elementwise.cu", "g2b_cache_write",
            [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_int, c_void_p])
    if k.dtype != cache_pages.dtype or v.dtype != cache_pages.dtype:
        raise KernelError("cache_write: k, v and the cache must have one dtype")
    _call(f, _ptr(k.contiguous()), _ptr(v.contiguous()), _code(k.dtype), k.shape[0], n_kv_heads,
          head_dim, _ptr(tok_pos), _ptr(tok_seq), _ptr(page_table), page_table.shape[1],
          _ptr(cache_pages), page_size, _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int, limit: float = 0.0, alpha: float = 1.0) -> None:
    """out[t, i] = silu(g_i) * u_i from a fused projection whose columns alternate
    ``block`` gates and ``block`` ups.  ``limit`` > 0: the capped form, g = min(g, limit),
    u = clamp(u, -limit, limit), out = g * sigmoid(alpha * g) * (u + 1)."""
    T, I = out.shape
    f = _fn("elementwise.cu", "g2b_swiglu",
            [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_float, c_void_p])
    _call(f, _ptr(gate_up), _code(gate_up.dtype), T, I, block, _ptr(out), float(limit), float(alpha), _stream())


def norm_shift(x32, w, mu, kept, ctx, eps: float, h_out, hs_out) -> None:
    """RMS norm of every row of the stream with a token shift: ``h_out`` = w * x / rms(x) and
    ``hs_out`` = h + (h_prev - h) * mu, h_prev the normed row of the token before in the sequence
    (``kept`` [slots, H] float32 holds it between steps and is brought up to date; zeros in front of
    position 0).  32-bit arithmetic; both outputs in the compute type."""
    _need(x32, torch.float32, "x")
    _need(mu, torch.float32, "shift weights")
    _need(kept, torch.float32, "kept rows")
    if w is not None:
        _need(w, torch.float32, "norm weight")
    if h_out.dtype != hs_out.dtype or not h_out.is_contiguous() or not hs_out.is_contiguous():
        raise KernelError("norm_shift: both outputs contiguous and of one dtype")
    T, H = x32.shape
    f = _fn("elementwise.cu", "g2b_norm_shift",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
             c_void_p, c_void_p, c_int, c_void_p])
    _call(f, _ptr(x32), _ptr(w), _ptr(mu), _ptr(kept), _ptr(ctx.tok_seq), _ptr(ctx.tok_pos), _ptr(ctx.seq_slots),
          _ptr(ctx.seq_meta), T, H, float(eps),
          _ptr(h_out), _ptr(hs_out), _code(h_out.dtype), _stream())


def advance_positions(tok_pos: torch.Tensor, n: int) -> None:
    f = _fn("elementwise.cu", "g2b_advance_positions", [c_void_p, c_int, c_void_p])
    _call(f, _ptr(tok_pos), n, _stream())


def rewind_step(tok_pos: torch.Tensor, n: int, seq_state: Optional[torch.Tensor], slots: Optional[torch.Tensor],
                undo_draw: bool, undo_recent: bool = False) -> None:
    """Takes back the device-side bookkeeping of one decode step (positions; the draw
    counters of the sampling records when that step sampled with a random number; the count
    of recent ids when it added one to the sequences' rings)."""
    f = _fn("elementwise.cu", "g2b_rewind_step",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    words = seq_state.shape[1] if seq_state is not None else 0
    _call(f, _ptr(tok_pos), n, _ptr(seq_state), words, _ptr(slots), 1 if undo_draw else 0,
          1 if undo_recent else 0, _stream())


# ---------------------------------------------------------------------------
# stream_ops.cu: the parts around the products of a gated layer with a latent cache
# ---------------------------------------------------------------------------
def embed_pair_norm(table, pairs, ids, ctx, ring, norm_w, eps, scale, buckets, mul_prev, mul_cur,
                    out) -> None:
    """out[t] = rmsnorm(table[ids[t]] * scale + pairs[row_t]) * norm_w as float32, row_t a hash of
    the previous and the current token (``buckets`` for a sequence's first token).  ``ring``
    int32 [slots, 2]: the last token of every sequence, by position parity."""
    from ctypes import c_longlong
    _need(ids, torch.int32, "ids")
    _need(out, torch.float32, "out")
    _need(ring, torch.int32, "ring")
    _need(norm_w, torch.float32, "norm weight")
    if pairs.dtype != table.dtype or pairs.shape[1] != table.shape[1] or pairs.shape[0] != buckets + 1:
        raise KernelError("embed_pair_norm: the pair table must be [buckets + 1, width] in the table's dtype")
    V, H = table.shape
    f = _fn("stream_ops.cu", "g2b_embed_pair_norm",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_longlong, c_longlong, c_longlong,
             c_float, c_void_p])
    _call(f, _ptr(table), _ptr(pairs), _code(table.dtype), _ptr(ids), _ptr(ctx.tok_pos), _ptr(ctx.tok_seq),
          _ptr(ctx.seq_slots), _ptr(ctx.seq_meta), _ptr(ring), _ptr(norm_w), _ptr(out), out.shape[0], H, V,
          float(scale), int(buckets), int(mul_prev), int(mul_cur), float(eps), _stream())


def canon_conv(h, w32, ring, ctx, out) -> None:
    """out = h + causal convolution of h over time per channel; w32 float32 [taps, width] (the
    oldest tap first); ``ring`` [slots, taps, width]: the rows before the step, by position mod taps."""
    _need(w32, torch.float32, "convolution weight")
    if ring.dtype != h.dtype or out.dtype != h.dtype:
        raise KernelError("canon_conv: input, output and ring must have one dtype")
    T, H = h.shape
    f = _fn("stream_ops.cu", "g2b_canon_conv",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
             c_int, c_void_p])
    _call(f, _ptr(h), _ptr(w32), _ptr(ring), _code(h.dtype), _ptr(ctx.tok_pos), _ptr(ctx.tok_seq),
          _ptr(ctx.seq_slots), _ptr(out), T, H, w32.shape[0], _stream())


def norm_canon_single(x32, norm_w, eps, w32, ring, ctx, h_out, u_out, add=None) -> None:
    """A step of one token per sequence: h_out = rmsnorm(x32) * norm_w, u_out = h + convolution of h
    (w32 float32 [taps, width]) with the earlier rows in ``ring``, and h into the ring at each token's
    position; one launch.  ``add`` = (y32, gate, bias): x32 += y32 * sigmoid(gate + bias) first (a gated
    addition that the layer in front left to this launch)."""
    _need(x32, torch.float32, "x")
    _need(norm_w, torch.float32, "norm weight")
    _need(w32, torch.float32, "convolution weight")
    if ring.dtype != h_out.dtype or u_out.dtype != h_out.dtype or not (h_out.is_contiguous() and u_out.is_contiguous()):
        raise KernelError("norm_canon_single: outputs and ring must have one dtype")
    T, H = x32.shape
    f = _fn("stream_ops.cu", "g2b_norm_canon_single",
            [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    y = g = b = None
    if add is not None:
        y, g, b = add
        _need(y, torch.float32, "y")
        if g.dtype != h_out.dtype or g.stride(1) != 1:
            raise KernelError("norm_canon_single: the gate must have the outputs' dtype and dense rows")
    _call(f, _ptr(x32), _ptr(norm_w), float(eps), _ptr(w32), _ptr(ring), _code(h_out.dtype), _ptr(ctx.tok_pos),
          _ptr(ctx.tok_seq), _ptr(ctx.seq_slots), _ptr(h_out), _ptr(u_out), T, H, w32.shape[0], _ptr(y), _ptr(g),
          g.stride(0) if g is not None else 0, _ptr(b), _stream())


def latent_keep(d, norm_w, eps, pages, h, ring, taps, ctx) -> None:
    """Writes rmsnorm(d) * norm_w (d [T, rank], a view with any row stride; None: nothing) into
    the latent pages at the tokens' positions, and the last ``taps - 1`` rows of ``h`` of every
    sequence into ``ring`` (None: nothing)."""
    f = _fn("stream_ops.cu", "g2b_latent_keep",
            [c_void_p, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_void_p,
             c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    if d is None and ring is None:
        return
    ref = d if d is not None else h
    if d is not None:
        _need(norm_w, torch.float32, "latent norm weight")
        if d.stride(1) != 1 or pages.dtype != d.dtype:
            raise KernelError("latent_keep: the latents must be rows of the cache's dtype")
    if ring is not None and (ring.dtype != h.dtype or not h.is_contiguous()):
        raise KernelError("latent_keep: ring and rows must have one dtype")
    _call(f, _ptr(d), d.stride(0) if d is not None else 0, d.shape[1] if d is not None else 0,
          _ptr(norm_w), float(eps), _ptr(pages), _ptr(ctx.page_table) if d is not None else None,
          ctx.page_table.shape[1] if d is not None else 0, ctx.page_size, _ptr(h) if ring is not None else None, _ptr(ring),
          h.shape[1] if ring is not None else 0, int(taps), _code(ref.dtype), _ptr(ctx.tok_pos),
          _ptr(ctx.tok_seq), _ptr(ctx.seq_slots), ref.shape[0], _stream())


def head_product(x, w, out, heads: int, expand: bool, gate=None) -> None:
    """One small matrix per head, w [heads * n, r].  ``expand`` False: out[t, h] = w_h^T x[t, h]
    (x has n values per head, out r); True: out[t, h] = w_h x[t, h] (x has r per head, out n),
    times sigmoid(gate[t, h]) when ``gate`` [T, heads] is given.  Views with row strides are taken."""
    n, r = w.shape[0] // heads, w.shape[1]
    if x.dtype != w.dtype or out.dtype != w.dtype or not w.is_contiguous():
        raise KernelError("head_product: x, w and out must have one dtype, w contiguous")
    if x.stride(1) != 1 or out.stride(1) != 1 or (gate is not None and (gate.stride(1) != 1 or gate.dtype != x.dtype)):
        raise KernelError("head_product: innermost strides must be 1")
    f = _fn("stream_ops.cu", "g2b_head_product",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
             c_int, c_int, c_void_p])
    _call(f, _ptr(x), x.stride(0), _ptr(w), _ptr(gate), gate.stride(0) if gate is not None else 0,
          _ptr(out), out.stride(0), x.shape[0], heads, n, r, 1 if expand else 0, _code(x.dtype), _stream())


def head_gate(o, gate, heads: int) -> None:
    """o[t, h, :] *= sigmoid(gate[t, h]) in place; o [T, heads * n] contiguous."""
    if not o.is_contiguous() or gate.dtype != o.dtype or gate.stride(1) != 1:
        raise KernelError("head_gate: o contiguous, gate of o's dtype")
    f = _fn("stream_ops.cu", "g2b_head_gate", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _call(f, _ptr(o), _ptr(gate), gate.stride(0), o.shape[0], heads, o.shape[1] // heads, _code(o.dtype), _stream())


def gated_add(x32, y32, g, bias, norm_w=None, eps: float = 0.0, normed=None) -> None:
    """x32 += y32 * sigmoid(g + bias) row by row (g a view with any row stride); with ``normed``
    also normed = rmsnorm(x32) * norm_w of the new rows."""
    _need(x32, torch.float32, "x")
    _need(y32, torch.float32, "y")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    if g.stride(1) != 1 or (normed is not None and (normed.dtype != g.dtype or not normed.is_contiguous())):
        raise KernelError("gated_add: gate rows must be dense, normed of the gate's dtype")
    if norm_w is not None:
        _need(norm_w, torch.float32, "norm weight")
    T, H = x32.shape
    f = _fn("stream_ops.cu", "g2b_gated_add",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_float, c_void_p,
             c_int, c_void_p])
    _call(f, _ptr(x32), _ptr(y32), _ptr(g), g.stride(0), _ptr(bias), T, H, _ptr(norm_w), float(eps),
          _ptr(normed), _code(g.dtype), _stream())


def xielu(z, pq32, out) -> None:
    """out = a z^2 + z/2 for z > 0, (1/2 + b)(exp(z) - 1 - z) + z/2 otherwise, a = softplus(pq[0]),
    b = softplus(pq[1]); z a view [T, F] with any row stride, out [T, F] contiguous."""
    _need(pq32, torch.float32, "activation parameters")
    if z.stride(1) != 1 or out.dtype != z.dtype or not out.is_contiguous():
        raise KernelError("xielu: dense rows of one dtype")
    f = _fn("stream_ops.cu", "g2b_xielu", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _call(f, _ptr(z), z.stride(0), _ptr(pq32), _ptr(out), z.shape[0], z.shape[1], _code(z.dtype), _stream())


# ---------------------------------------------------------------------------
# random_init.cu
# ---------------------------------------------------------------------------
def philox_normal(out: torch.Tensor, seed: int, tensor_index: int, scale_vector: bool, std: float) -> None:
    """Fills ``out`` (float32 or bfloat16, contiguous) in place with N(0, std), or with
    1 + N(0, std) for a scale vector; element i gets the value of (seed, tensor_index, i)."""
    if not out.is_contiguous():
        raise KernelError("philox_normal: the tensor must be contiguous")
    from ctypes import c_longlong, c_uint
    f = _fn("random_init.cu", "g2b_philox_normal",
            [c_void_p, c_int, c_longlong, c_ulonglong, c_uint, c_int, c_float, c_void_p])
    _call(f, _ptr(out), _code(out.dtype), out.numel(), int(seed) & 0xFFFFFFFFFFFFFFFF,
          int(tensor_index) & 0xFFFFFFFF, 1 if scale_vector else 0, float(std), _stream())


# ---------------------------------------------------------------------------
# matrix products
# ---------------------------------------------------------------------------
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out (=|+=) a @ w.T in true float32 arithmetic.  a [M,K], w [N,K], out [M,N];
    accumulate needs a float32 out."""
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: shapes a{list(a.shape)} w{list(w.shape)} out{list(out.shape)}")
    if accumulate:
        _need(out, torch.float32, "accumulated output")
        epi = EPI_ACCUM_F32
    else:
        epi = EPI_STORE_F32 if out.dtype == torch.float32 else EPI_STORE_BF16
        _code(out.dtype)
    f = _fn("gemm_simt.cu", "g2b_gemm_simt",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
             c_int, c_void_p])
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm: innermost strides must be 1")
    _call(f, _ptr(a), _code(a.dtype), _ptr(w), _code(w.dtype), _ptr(out), M, N, K, a.stride(0),
          w.stride(0), out.stride(0), epi, _stream())


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """The product a layer asks for; picks the kernel from the dtypes and sizes.  Anything
    that is not all-bfloat16 runs on the float32 kernel (true 32-bit arithmetic)."""
    if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        if (_bf16 or _bf16_mod()).linear_bf16(a, w, out, accumulate):
            return
    gemm_simt(a, w, out, accumulate)


def product_notices(what: str, w: Optional[torch.Tensor], compute_dtype: torch.dtype) -> list:
    """Why products with the matrix ``w`` will run on the 32-bit FFMA kernel although the
    model computes in bfloat16: one line per reason, for the notice printed when a model is
    built (the result is right either way; the speed is not the same)."""
    if w is None or compute_dtype != torch.bfloat16:
        return []
    if w.dtype != torch.bfloat16:
        return [f"{what}: the matrix is kept in {str(w.dtype).replace('torch.', '')} as stored, so its "
                "products run on the 32-bit FFMA kernel, not on the tensor cores"]
    if w.shape[1] % 8 or w.stride(0) % 8 or w.data_ptr() % 16:
        return [f"{what}: K = {w.shape[1]} is no multiple of 8, so its products run on the 32-bit "
                "FFMA kernel, not on the tensor cores"]
    return []


def attention_notices(what: str, head_dim: int, page_size: int, compute_dtype: torch.dtype) -> list:
    if compute_dtype != torch.bfloat16:
        return []
    from . import kernels_bf16
    if head_dim not in kernels_bf16.FAST_HEAD_SIZES or page_size != 64:
        sizes = " and ".join(str(h) for h in kernels_bf16.FAST_HEAD_SIZES)
        return [f"{what}: head size {head_dim} runs on the 32-bit attention kernel (the tensor-core "
                f"kernels take head sizes {sizes})"]
    return []


# ---------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------
def attn_generic(q, out, cache_pages, tok_pos, tok_seq, page_table, n_heads, n_kv_heads,
                 head_dim, page_size, window, scale, sink=None, planes: int = 2, gate=None, chunk: int = 0,
                 pooled=None, pool: int = 0, softcap: float = 0.0, keep_first: int = 0, v_heads: int = 0) -> None:
    """Causal attention of every token of the step over its sequence's cache pages,
    32-bit arithmetic; q [T, n_heads*head_dim] (rows may lie further apart: columns of a wider
    buffer), out [T, n_heads*head_dim] contiguous.  ``sink`` (float32 [n_heads]): one more
    term exp(sink_h) in each head's softmax denominator.  ``planes`` = 1: the pages hold one
    panel per kv head that is read as keys and as values.  ``gate`` [T, n_heads] (rows may lie
    further apart): every head's output is multiplied by the sigmoid of its gate.  ``chunk`` > 0:
    a token sees the keys of its own chunk of that many positions only (counted from position 0).
    ``pool`` > 0 with ``pooled`` [pages, 2, kv heads, rows, head_dim] (and a window): in front of the
    window a token also sees the mean key and value of every block of ``pool`` positions that lies
    wholly before the window, in the same softmax.  ``softcap`` > 0: scores become softcap * tanh(score /
    softcap).  ``keep_first`` > 0 (with a window): the first that many positions stay visible behind the
    window.  ``v_heads`` (a divisor of the kv heads): key head g reads the values of head g mod v_heads."""
    f = _fn("attn_generic.cu", "g2b_attn_generic",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
             c_int, c_int, c_float, c_int, c_int, c_void_p])
    if pool and (pooled is None or pooled.dtype != q.dtype):
        raise KernelError("attention: pooled blocks need their store, of q's dtype")
    if q.dtype != cache_pages.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q, out and the cache must have one dtype")
    if q.stride(1) != 1 or not out.is_contiguous() or (gate is not None and (gate.stride(1) != 1 or gate.dtype != q.dtype)):
        raise KernelError("attention: q and gate need dense rows, out must be contiguous, gate of q's dtype")
    if sink is not None:
        _need(sink, torch.float32, "sink")
    _call(f, _ptr(q), _ptr(out), _code(q.dtype), _ptr(cache_pages), _ptr(tok_pos), _ptr(tok_seq),
          _ptr(page_table), page_table.shape[1], q.shape[0], n_heads, n_kv_heads, head_dim,
          page_size, window, scale, _ptr(sink), planes, q.stride(0), _ptr(gate),
          gate.stride(0) if gate is not None else 0, int(chunk), _ptr(pooled) if pool else None, int(pool),
          pooled.shape[3] if pool else 0, float(softcap), int(keep_first), int(v_heads), _stream())


def attention(q, out, cache_pages, ctx, n_heads, n_kv_heads, head_dim, page_size, window,
              scale, sink=None, planes: int = 2, gate=None, chunk: int = 0, pooled=None, pool: int = 0,
              softcap: float = 0.0, keep_first: int = 0, v_heads: int = 0) -> None:
    """Attention of a step: the tensor-core kernels when they take the case, else the
    32-bit kernel.  ``q`` and ``gate`` may be column ranges of a wider buffer.  ``pool``, ``pooled``:
    mean keys and values of whole blocks in front of the window (``attn_generic``).  ``softcap``,
    ``keep_first``, ``v_heads``: as ``attn_generic``."""
    if pool:
        if q.dtype == torch.bfloat16 and (_bf16 or _bf16_mod()).attention_pooled_bf16(
                q, out, cache_pages, pooled, ctx, n_heads, n_kv_heads, head_dim, page_size, window, pool, scale):
            return
        attn_generic(q, out, cache_pages, ctx.tok_pos, ctx.tok_seq, ctx.page_table, n_heads, n_kv_heads, head_dim,
                     page_size, window, scale, sink, planes, gate, chunk, pooled, pool)
        return
    if q.dtype == torch.bfloat16:
        if (_bf16 or _bf16_mod()).attention_bf16(q, out, cache_pages, ctx, n_heads, n_kv_heads, head_dim,
                                       page_size, window, scale, sink, planes, gate, chunk,
                                       softcap=softcap, keep_first=keep_first, v_heads=v_heads):
            return
    attn_generic(q, out, cache_pages, ctx.tok_pos, ctx.tok_seq, ctx.page_table, n_heads,
                 n_kv_heads, head_dim, page_size, window, scale, sink, planes, gate, chunk,
                 softcap=softcap, keep_first=keep_first, v_heads=v_heads)


def normed_product(x32, eps, w, out, gate_block=None) -> bool:
    """out = rmsnorm_without_weight(x32) @ w.T (or its SiLU gate) in one kernel; False when no
    kernel takes the case (the caller then runs the norm and the product one after the other)."""
    if w.dtype == torch.bfloat16 and (gate_block is None or gate_block == 8):
        return (_bf16 or _bf16_mod()).normed_product(x32, eps, w, out, gate_block is not None)
    return False


def gate_up_fused(h, w_gate_up, mid, block) -> bool:
    """silu(gate) * up computed inside the product's epilogue; False when no kernel takes
    the case (the caller then runs the product and ``swiglu`` separately)."""
    if h.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16:
        return (_bf16 or _bf16_mod()).gate_up_bf16(h, w_gate_up, mid, block)
    return False


# ---------------------------------------------------------------------------
# sampling.cu
# ---------------------------------------------------------------------------
def sample_rows(logits, temperature, seq_state, slots, out_ids) -> None:
    """Greedy (temperature <= 0) or temperature sampling of one id per row of float32
    logits; random numbers come from the per-slot records."""
    _need(logits, torch.float32, "logits")
    _need(out_ids, torch.int32, "out_ids")
    R, V = logits.shape
    if temperature <= 0.0 and V >= 4096:
        # greedy over a large vocabulary: many blocks per row, then one
        n = max(R, 64) * 64
        scratch = (_scratch_buffer((logits.device, "argmax values"), n, torch.float32),
                   _scratch_buffer((logits.device, "argmax indices"), n, torch.int32))
        f = _fn("sampling.cu", "g2b_argmax_rows",
                [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
        _call(f, _ptr(logits), R, V, logits.stride(0), _ptr(scratch[0]), _ptr(scratch[1]),
              _ptr(out_ids), _stream())
        count_launches(1)                          # the slices, then the winner among them
        return
    f = _fn("sampling.cu", "g2b_sample_rows",
            [c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    pieces = None
    if temperature > 0.0 and V >= 8192:
        # a large vocabulary: many blocks per row sum its pieces first
        pieces = _scratch_buffer((logits.device, "pieces"), max(R, 64) * 2048 * 2, torch.float32)
        count_launches(1)
    _call(f, _ptr(logits), R, V, logits.stride(0), temperature, _ptr(seq_state),
          seq_state.shape[1] if seq_state is not None else 0, _ptr(slots), _ptr(out_ids), _ptr(pieces),
          _stream())


def sample_filtered(logits, temperature, top_k, top_p, penalty, recent, recent_n, seq_state, slots,
                    out_ids, append: bool = False) -> None:
    """Repeat penalty, top-k, top-p, then temperature sampling; logits are changed in
    place by the penalty.  recent int32 [R, n], recent_n int32 [R]; or ``recent=None``: every
    row's recent ids are those in its sequence's record (``seq_state[slots[row]]``), to which
    the chosen id is added when ``append`` is set."""
    _need(logits, torch.float32, "logits")
    _need(out_ids, torch.int32, "out_ids")
    R, V = logits.shape
    if recent is not None:
        _need(recent, torch.int32, "recent")
        _need(recent_n, torch.int32, "recent_n")
        if recent.shape[0] < R or recent_n.shape[0] < R:
            raise KernelError("sample_filtered: recent and recent_n need a row per row of logits")
    f = _fn("sampling.cu", "g2b_sample_filtered",
            [c_void_p, c_int, c_int, c_int, c_float, c_int, c_float, c_float, c_void_p, c_int,
             c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    cand = None
    if temperature > 0.0 and 0 < top_k <= 256 and V >= 8192:
        # a small top_k over a large vocabulary: many blocks per row list the candidates first
        words = _fn("sampling.cu", "g2b_sample_filtered_scratch_words", [c_int])
        cand = _scratch_buffer((logits.device, "filter"), int(words(max(R, 64))), torch.int32)
        count_launches(1)
    _call(f, _ptr(logits), R, V, logits.stride(0), temperature, top_k, top_p, penalty,
          _ptr(recent), recent.shape[1] if recent is not None else 0, _ptr(recent_n),
          _ptr(seq_state), seq_state.shape[1] if seq_state is not None else 0, _ptr(slots),
          _ptr(out_ids), 1 if append else 0, _ptr(cand), _stream())


def recent_set(seq_state, slots, rows) -> None:
    """Starts the recent-id rings of the given slots: rows int32 [n, 65] = count, ids (oldest
    first); the repeat penalty of later ``sample_filtered`` calls without ``recent`` reads them."""
    _need(slots, torch.int32, "slots")
    _need(rows, torch.int32, "rows")
    if rows.dim() != 2 or rows.shape[1] != 65 or rows.shape[0] < slots.shape[0]:
        raise KernelError("recent_set: rows must be [n, 65]")
    f = _fn("sampling.cu", "g2b_recent_set", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p])
    _call(f, _ptr(seq_state), seq_state.shape[1], _ptr(slots), _ptr(rows), slots.shape[0], _stream())


def seed_slots(seq_state, slots, streams, seed: int) -> None:
    """Starts the random stream of each given slot: key = seed, stream id, zero draws."""
    f = _fn("sampling.cu", "g2b_seed_slots",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_ulonglong, c_void_p])
    _call(f, _ptr(seq_state), seq_state.shape[1], _ptr(slots), _ptr(streams), slots.shape[0],
          seed & 0xFFFFFFFFFFFFFFFF, _stream())


# ---------------------------------------------------------------------------
# seq_mix.cu: mixers with a matrix state, their short convolution, a wide attention prologue
# ---------------------------------------------------------------------------
def _dense_rows(t: torch.Tensor, what: str) -> int:
    if t.stride(1) != 1:
        raise KernelError(f"{what}: rows must be dense (they may lie apart)")
    return t.stride(0)


def proj_norm_rope_cache(qkv, bias, n_heads, n_kv_heads, qk_dim, v_dim, q_w, k_w, eps, rope, rotary_dim,
                         interleaved, ctx, cache_pages, page_size, q_out, v_norm_eps: float = 0.0,
                         norm_per_head: bool = False, unit_eps: float = 0.0, n_v_heads: Optional[int] = None) -> None:
    """q, k, v side by side in ``qkv`` [T, nh*D + nkv*D + nkv*V] (+ ``bias``, float32); RMS norm over
    ALL of q and over all of k (weights ``q_w`` [nh*D], ``k_w`` [nkv*D]; None: no norm); rotation by
    the step's ``rope`` table, pairs (i, i + r/2) or, ``interleaved``, (2i, 2i + 1); q to ``q_out``
    [T, nh*hd] and k, v into the pages, heads zero-filled to hd = max(D, V).  ``v_norm_eps`` > 0: every
    value head is divided by its root mean square (that eps inside the root) before it is stored.
    ``norm_per_head``: the norm runs over every head of q and k by itself, the weights ``q_w``, ``k_w`` [D]
    shared by the heads.  ``unit_eps`` > 0: after the rotation every head of q and k is divided by its
    root mean square (that eps inside the root, no weight).  ``n_v_heads``: fewer value heads than key
    heads (``qkv`` then ends with that many; the other value panels of the pages stay unused).
    ``n_kv_heads`` 0 (``cache_pages`` None): q alone, for a layer that reads another layer's pages."""
    f = _fn("seq_mix.cu", "g2b_proj_norm_rope_cache",
            [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
             c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_float,
             c_int, c_float, c_int, c_void_p])
    if q_out.dtype != qkv.dtype or (cache_pages is not None and cache_pages.dtype != qkv.dtype) or not q_out.is_contiguous():
        raise KernelError("proj_norm_rope_cache: q_out and the cache must have the input's dtype")
    for t in (bias, q_w, k_w):
        if t is not None:
            _need(t, torch.float32, "bias / norm weight")
    _call(f, _ptr(qkv), _code(qkv.dtype), _dense_rows(qkv, "qkv"), qkv.shape[0], _ptr(bias), n_heads, n_kv_heads,
          qk_dim, v_dim, _ptr(q_w), _ptr(k_w), eps, _ptr(rope), rotary_dim, 1 if interleaved else 0,
          _ptr(ctx.tok_pos), _ptr(ctx.tok_seq), _ptr(ctx.page_table), ctx.page_table.shape[1],
          _ptr(cache_pages), page_size, _ptr(q_out), float(v_norm_eps), 1 if norm_per_head else 0, float(unit_eps),
          n_kv_heads if n_v_heads is None else int(n_v_heads), _stream())


def rotate_heads(x, heads, head_dim, rope, rotary_dim, interleaved, scale: float = 1.0) -> None:
    """In place: the first ``rotary_dim`` entries of every head of x [T, heads*head_dim] (rows may lie
    apart) turn by the step's ``rope`` table; then everything times ``scale``."""
    f = _fn("seq_mix.cu", "g2b_rotate_heads",
            [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_float, c_void_p])
    _call(f, _ptr(x), _code(x.dtype), _dense_rows(x, "x"), x.shape[0], heads, head_dim, _ptr(rope), rotary_dim,
          1 if interleaved else 0, scale, _stream())


def short_conv(x, w32, ring, ctx, out, act: bool = True, bias=None) -> None:
    """out_t = act(bias[c] + sum_j w32[j, c] * x_{t - taps + 1 + j}[c]) per channel, act = SiLU; ``w32`` float32
    [taps, C]; ``ring`` [slots, taps, C] holds every sequence's last input rows by position mod taps
    and is brought up to date (in the same launch for a step of one token per sequence)."""
    taps, C = w32.shape
    _need(w32, torch.float32, "convolution weights")
    if out.dtype != x.dtype or (ring is not None and ring.dtype != x.dtype):
        raise KernelError("short_conv: input, output and ring must have one dtype")
    f = _fn("seq_mix.cu", "g2b_short_conv",
            [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p])
    if bias is not None:
        _need(bias, torch.float32, "convolution bias")
    _call(f, _ptr(x), _code(x.dtype), _dense_rows(x, "x"), _ptr(w32), _ptr(ring), taps, C, x.shape[0], ctx.n_seqs,
          _ptr(ctx.tok_pos), _ptr(ctx.tok_seq), _ptr(ctx.seq_slots), _ptr(ctx.seq_meta), 1 if act else 0,
          _ptr(out), _dense_rows(out, "out"), _ptr(bias), _stream())
    if ctx.seq_meta is not None and taps > 1:
        count_launches(1)


def state_scan(q, k, v, state, ctx, out32, heads, qk_heads, qk_dim, v_dim, *, decay=None, ab=None, a_log=None,
               dt_bias=None, rope=None, rotary_dim: int = 0, interleaved: bool = False, q_scale: float = 1.0,
               k_scale: float = 1.0, unit_eps: Optional[float] = None, gates=None, ones_column: bool = False) -> None:
    """The recurrence of a mixer with a matrix state per head, over the step's tokens in order;
    ``state`` float32 [slots, heads, v_dim, qk_dim] is read and left up to date.  ``decay`` (float32
    [heads]): S = a S + k v^T.  Otherwise ``ab`` (float32 [T, 2*heads]: x then y), ``a_log``, ``dt_bias``:
    S = g S with g = exp(-exp(a_log) softplus(x + dt_bias)); u = sigmoid(y) (v - S^T k); S += k u^T.
    Or ``gates`` (float32 [T, 2*heads]: a decay g, then a strength s, per token and head, as
    ``scan_gates_step`` / ``scan_gates_max`` make them): S = g S + s k v^T.
    Either way o = S^T q, float32 into ``out32`` [T, heads*v_dim].  q and k first turn by ``rope``
    (or, with ``unit_eps``, are divided by sqrt(sum x^2 + unit_eps)), then take their scales.
    ``ones_column``: every head carries one more column whose value is 1 at every token (the weighted
    sum of the keys); state and output then have ``v_dim + 1`` columns a head."""
    T = q.shape[0]
    _need(state, torch.float32, "state")
    _need(out32, torch.float32, "scan output")
    mode = 0 if decay is not None else (2 if gates is not None else 1)
    if gates is not None:
        ab = gates
    cols = v_dim + (1 if ones_column else 0)
    if tuple(state.shape[1:]) != (heads, cols, qk_dim) or tuple(out32.shape) != (T, heads * cols):
        raise KernelError(f"state_scan: state {tuple(state.shape)} or output {tuple(out32.shape)} do not fit "
                          f"{heads} heads of {cols} columns of {qk_dim}")
    for t in (decay, ab, a_log, dt_bias):
        if t is not None:
            _need(t, torch.float32, "decay inputs")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise KernelError("state_scan: q, k and v must have one dtype")
    common = [mode, _code(q.dtype), _ptr(q), _dense_rows(q, "q"), _ptr(k), _dense_rows(k, "k"), _ptr(v),
              _dense_rows(v, "v"), heads, qk_heads, qk_dim, v_dim, _ptr(rope), rotary_dim, 1 if interleaved else 0,
              q_scale, k_scale, 0 if unit_eps is None else 1, unit_eps or 0.0, _ptr(decay), _ptr(ab), _ptr(a_log),
              _ptr(dt_bias), _ptr(state)]
    types = [c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
             c_int, c_int, c_float, c_float, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
    if ctx.seq_meta is not None and T > ctx.n_seqs:
        # a prompt step: q and k are prepared once (rotation or unit norm, scales; float), then a scan
        # that fetches the next tokens while it works on the ones it has
        qf = ctx.workspace.buffer("scan.q", (T, qk_heads * qk_dim), torch.float32)
        kf = ctx.workspace.buffer("scan.k", (T, qk_heads * qk_dim), torch.float32)
        f = _fn("seq_mix.cu", "g2b_state_scan_prompt",
                types + [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
        _call(f, *common, _ptr(ctx.seq_meta), T, ctx.n_seqs, _ptr(qf), _ptr(kf), _ptr(out32),
              1 if ones_column else 0, _stream())
        count_launches(1)
        return
    f = _fn("seq_mix.cu", "g2b_state_scan",
            types + [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p])
    _call(f, *common, _ptr(ctx.tok_pos), _ptr(ctx.seq_slots), _ptr(ctx.seq_meta), T, ctx.n_seqs,
          _ptr(out32), 1 if ones_column else 0, _stream())


def scan_gates_step(x, a_log, dt_bias, gates) -> None:
    """Decay and strength of a state-space head from its step size: dt = softplus(x + dt_bias),
    g = exp(-exp(a_log) dt), s = dt; x [T, heads] (columns of a wider buffer), ``gates`` float32
    [T, 2*heads]: g, then s."""
    _need(gates, torch.float32, "gates")
    _need(a_log, torch.float32, "a_log")
    _need(dt_bias, torch.float32, "dt_bias")
    T, H = x.shape
    f = _fn("seq_mix.cu", "g2b_scan_gates_step",
            [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _call(f, _ptr(x), _code(x.dtype), _dense_rows(x, "x"), _ptr(a_log), _ptr(dt_bias), T, H, _ptr(gates), _stream())


def scan_gates_max(x_i, x_f, b_i, b_f, cap: float, m_state, ctx, gates, m_out) -> None:
    """Exponential gates under a running maximum: i = cap tanh((x_i + b_i) / cap),
    f = logsigmoid(cap tanh((x_f + b_f) / cap)), m' = max(f + m, i), g = exp(f + m - m'),
    s = exp(i - m'); ``m_state`` float32 [slots, heads] holds m between steps (from 0) and is left
    up to date; ``gates`` float32 [T, 2*heads]: g, then s; ``m_out`` float32 [T, heads]: m' per token."""
    for t, what in ((gates, "gates"), (m_out, "m_out"), (m_state, "m_state"), (b_i, "b_i"), (b_f, "b_f")):
        _need(t, torch.float32, what)
    if x_i.dtype != x_f.dtype or x_i.stride(0) != x_f.stride(0):
        raise KernelError("scan_gates_max: both gate inputs are columns of one buffer")
    H = x_i.shape[1]
    f = _fn("seq_mix.cu", "g2b_scan_gates_max",
            [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_void_p, c_void_p])
    _call(f, _ptr(x_i), _ptr(x_f), _code(x_i.dtype), _dense_rows(x_i, "x_i"), _ptr(b_i), _ptr(b_f), float(cap), H,
          _ptr(m_state), _ptr(ctx.seq_slots), _ptr(ctx.seq_meta), ctx.n_seqs, _ptr(gates), _ptr(m_out), _stream())


def state_readout(o32, heads, v_dim, out, *, stored_cols: Optional[int] = None, m=None, den_eps: float = 0.0,
                  skip_x=None, skip_w=None, gate=None, gate_act: str = "silu", gate_first: bool = False,
                  group: Optional[int] = None, eps: float = 0.0, w=None) -> None:
    """What a scan reads out, made ready for the output product, 32-bit: with ``m`` [T, heads] every
    head is divided by max(|its column v_dim|, exp(-m)) + den_eps; ``skip_w`` [heads] times ``skip_x``
    [T, heads*v_dim] is added; ``gate_first``: times act(gate); then every ``group`` neighbouring
    outputs (default: a head) are divided by their root mean square (``eps`` inside the root), times
    ``w`` (one per output, or one head's worth shared by all), times act(gate) if not before.
    act: "silu" or "sigmoid".  ``out`` [T, heads*v_dim] in the compute type."""
    _need(o32, torch.float32, "scan output")
    T = o32.shape[0]
    Vs = int(stored_cols or v_dim)
    if gate_act not in ("silu", "sigmoid"):
        raise KernelError(f"state_readout: gate activation {gate_act!r}")
    for t in (m, skip_w, w):
        if t is not None:
            _need(t, torch.float32, "read-out inputs")
    for t in (skip_x, gate):
        if t is not None and t.dtype != out.dtype:
            raise KernelError("state_readout: skip input and gate must have the output's dtype")
    f = _fn("seq_mix.cu", "g2b_state_readout",
            [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_float, c_void_p, c_int, c_int, c_void_p, c_void_p])
    _call(f, _ptr(o32), T, heads, v_dim, Vs, _ptr(m), float(den_eps), _ptr(skip_x),
          _dense_rows(skip_x, "skip_x") if skip_x is not None else 0, _ptr(skip_w), _ptr(gate),
          _dense_rows(gate, "gate") if gate is not None else 0, 1 if gate_act == "sigmoid" else 0,
          1 if gate_first else 0, int(group or v_dim), float(eps), _ptr(w), w.numel() if w is not None else 0,
          _code(out.dtype), _ptr(out), _stream())


def pool_update(cache_pages, pooled_pages, ctx, n_kv_heads, head_dim, page_size, pool: int) -> None:
    """Every token of the step that ends a block of ``pool`` positions writes the mean of the block's
    keys and of its values (as the pages hold them) into ``pooled_pages`` [pages, 2, kv heads, rows,
    head_dim]: block b in the page of its first position, at row b - ceil(that page's first position / pool)."""
    if pooled_pages.dtype != cache_pages.dtype:
        raise KernelError("pool_update: both stores must have one dtype")
    f = _fn("seq_mix.cu", "g2b_pool_update",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
             c_void_p])
    _call(f, _ptr(cache_pages), _ptr(pooled_pages), _code(cache_pages.dtype), _ptr(ctx.tok_pos), _ptr(ctx.tok_seq),
          _ptr(ctx.page_table), ctx.page_table.shape[1], ctx.n_tokens, n_kv_heads, head_dim, page_size, int(pool),
          pooled_pages.shape[3], _stream())


def head_norm_gate(o32, heads, v_dim, w, eps, gate, out_scale, out) -> None:
    """out = o / sqrt(mean(o^2) + eps) per head (times ``w`` [v_dim], float32, if given), times
    silu(gate) (if given; [T, heads*v_dim], rows may lie apart), times ``out_scale``."""
    _need(o32, torch.float32, "scan output")
    if w is not None:
        _need(w, torch.float32, "head norm weight")
    f = _fn("seq_mix.cu", "g2b_head_norm_gate",
            [c_void_p, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p])
    if gate is not None and gate.dtype != out.dtype:
        raise KernelError("head_norm_gate: gate and output must have one dtype")
    _call(f, _ptr(o32), o32.shape[0], heads, v_dim, _ptr(w), eps, _ptr(gate),
          _dense_rows(gate, "gate") if gate is not None else 0, _code(out.dtype), out_scale, _ptr(out), _stream())


def gate_mul(o, head_dim, gate, heads, v_dim, out_scale, out) -> None:
    """out[t, h*v_dim + j] = o[t, h*head_dim + j] * sigmoid(gate[t, h*v_dim + j]) * out_scale."""
    f = _fn("seq_mix.cu", "g2b_gate_mul",
            [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    if out.dtype != o.dtype or (gate is not None and gate.dtype != o.dtype) or not o.is_contiguous():
        raise KernelError("gate_mul: one dtype, and a contiguous input")
    _call(f, _ptr(o), head_dim, _ptr(gate), _dense_rows(gate, "gate") if gate is not None else 0, _code(o.dtype),
          o.shape[0], heads, v_dim, out_scale, _ptr(out), _stream())


def norm_add(x32, y32, w, eps, cast_out=None) -> None:
    """x += y / sqrt(mean(y^2) + eps) * w (float32; ``w`` None: no weight); the new x once more,
    rounded, into ``cast_out``.  ``y32`` None: only the rounding."""
    _need(x32, torch.float32, "stream")
    if y32 is not None:
        _need(y32, torch.float32, "sublayer output")
    if w is not None:
        _need(w, torch.float32, "norm weight")
    f = _fn("seq_mix.cu", "g2b_norm_add",
            [c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p, c_int, c_void_p])
    _call(f, _ptr(x32), _ptr(y32), _ptr(w), eps, x32.shape[0], x32.shape[1], _ptr(cast_out),
          _code(cast_out.dtype) if cast_out is not None else F32, _stream())


def selective_scan(x, dt32, dt_bias, bc, a, skip, z, state, ctx, out, out_scale: float = 1.0) -> None:
    """A state-space recurrence with a decay per state entry, over the step's tokens in order:
    dt = softplus(dt32 + dt_bias); S[c, n] = exp(dt_c a[c, n]) S[c, n] + dt_c x_c B_n; y_c = sum_n S[c, n] C_n;
    out = (y + skip * x) * silu(z) * out_scale.  x, z [T, inner] and ``bc`` [T, 2N] (B, then C) in the
    compute type, rows may lie apart; ``dt32`` float32 [T, inner]; ``a`` float32 [inner, N] (negative);
    ``state`` float32 [slots, inner, N] is read and left up to date."""
    T, inner = x.shape
    N = a.shape[1]
    for t, what in ((dt32, "step sizes"), (dt_bias, "dt bias"), (a, "decay rates"), (skip, "skip"), (state, "state")):
        _need(t, torch.float32, what)
    if z.dtype != x.dtype or bc.dtype != x.dtype or out.dtype != x.dtype:
        raise KernelError("selective_scan: x, z, B/C and out must have one dtype")
    if tuple(state.shape[1:]) != (inner, N) or bc.shape[1] != 2 * N or tuple(a.shape) != (inner, N):
        raise KernelError(f"selective_scan: state {tuple(state.shape)}, B/C {tuple(bc.shape)} or rates {tuple(a.shape)} "
                          f"do not fit {inner} channels of {N} entries")
    f = _fn("seq_mix.cu", "g2b_selective_scan",
            [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p])
    _call(f, _ptr(x), _code(x.dtype), _dense_rows(x, "x"), _ptr(dt32), _dense_rows(dt32, "dt"), _ptr(dt_bias), _ptr(bc),
          _dense_rows(bc, "B/C"), _ptr(a), _ptr(skip), _ptr(z), _dense_rows(z, "z"), _ptr(state), _ptr(ctx.seq_slots),
          _ptr(ctx.seq_meta), T, ctx.n_seqs, inner, N, float(out_scale), _ptr(out), _dense_rows(out, "out"), _stream())


def diff_combine(a, heads: int, head_dim: int, v_dim: int, lam: float, eps: float, post: float, out) -> None:
    """Two attention maps per head, ``a`` [T, 2 * heads * head_dim] (all heads of the first map, then of
    the second; ``v_dim`` entries of a head in use): out[t, h] = (a1 - lam * a2) / sqrt(mean(.^2) + eps) *
    post, [T, heads * v_dim]."""
    if not a.is_contiguous() or not out.is_contiguous() or out.dtype != a.dtype:
        raise KernelError("diff_combine: contiguous tensors of one dtype")
    f = _fn("seq_mix.cu", "g2b_diff_combine",
            [c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p, c_void_p])
    _call(f, _ptr(a), _code(a.dtype), a.shape[0], heads, head_dim, v_dim, float(lam), float(eps), float(post), _ptr(out),
          _stream())


# ---------------------------------------------------------------------------
# moe.cu: a routed feed-forward
# ---------------------------------------------------------------------------
def moe_tile_rows() -> int:
    lib = load_unit("moe.cu")
    return int(lib.g2b_moe_tile_rows())


def moe_route(z32, correction, top: int, renormalise: bool, idx, weight, scale: float = 1.0, score: str = "softmax",
              groups: int = 1, keep: int = 1) -> None:
    """softmax over all experts of ``z32`` [T, N] (``score`` "sigmoid": every logit's sigmoid by itself);
    the ``top`` largest of score + correction chosen (``idx`` int32 [T, top]); ``weight`` float32 [T, top]
    their scores (divided by their sum + 1e-20 when ``renormalise``), times ``scale``.  ``groups`` > 1: the
    experts are that many equal groups of neighbours, a group counts as the sum of its two best scores,
    and only experts of the ``keep`` best groups can be chosen."""
    if score not in ("softmax", "sigmoid"):
        raise KernelError(f"moe_route: scores are 'softmax' or 'sigmoid', not {score!r}")
    _need(z32, torch.float32, "router logits")
    _need(idx, torch.int32, "idx")
    _need(weight, torch.float32, "weight")
    f = _fn("moe.cu", "g2b_moe_route", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                                        c_int, c_int, c_int, c_void_p])
    _call(f, _ptr(z32), _ptr(correction), z32.shape[0], z32.shape[1], top, 1 if renormalise else 0, _ptr(idx),
          _ptr(weight), float(scale), 1 if score == "sigmoid" else 0, int(groups), int(keep), _stream())


def moe_plan(idx, n_real: int, max_tiles: int, plan, row_pair, pair_row) -> None:
    """Groups the (token, choice) pairs of ``idx`` by expert; experts from ``n_real`` on get no rows."""
    f = _fn("moe.cu", "g2b_moe_plan", [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _call(f, _ptr(idx), idx.numel(), n_real, moe_tile_rows(), max_tiles, _ptr(plan), _ptr(row_pair), _ptr(pair_row),
          _stream())


def moe_gemm(a, row_pair, pairs_per_token: int, w, n_out: int, plan, n_real: int, max_tiles: int, swiglu: bool,
             out, blocked: bool = False) -> None:
    """Per expert e over its rows: out[row] = a[source of row] . w[e]^T; ``w`` [E, n_out (x2 with
    ``swiglu``: gate rows then up rows, or, ``blocked``, eight gates and eight ups in turn), K];
    ``row_pair`` None: row r reads a[r]."""
    if w.dtype != a.dtype:
        raise KernelError("moe_gemm: activations and expert matrices must have one dtype")
    f = _fn("moe.cu", "g2b_moe_gemm",
            [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int,
             c_void_p, c_int, c_int, c_void_p])
    _call(f, _ptr(a), _code(a.dtype), _dense_rows(a, "a"), _ptr(row_pair), pairs_per_token, _ptr(w), n_out,
          a.shape[1], _ptr(plan), n_real, max_tiles, 1 if swiglu else 0, _ptr(out),
          1 if out.dtype == torch.float32 else 0, 1 if blocked else 0, _stream())


def moe_gemv(a, row_pair, pairs_per_token: int, gather: bool, idx, w, n_out: int, plan, n_real: int, n_rows: int,
             swiglu: bool, out, blocked: bool = False) -> bool:
    """``moe_gemm`` for a step of few rows: a warp per four output columns of one row, the weight rows
    streamed with 16-byte loads.  ``gather``: row r reads a[pair / pairs_per_token], else a[r].  False
    when the sizes do not allow 16-byte loads (the caller then takes ``moe_gemm``)."""
    if w.dtype != a.dtype:
        raise KernelError("moe_gemv: activations and expert matrices must have one dtype")
    per = 8 if a.dtype == torch.bfloat16 else 4
    if a.shape[1] % per or a.stride(0) % per or a.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    f = _fn("moe.cu", "g2b_moe_gemv",
            [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
             c_int, c_void_p, c_int, c_int, c_void_p])
    _call(f, _ptr(a), _code(a.dtype), _dense_rows(a, "a"), _ptr(row_pair), pairs_per_token, 1 if gather else 0,
          _ptr(idx), _ptr(w), n_out, a.shape[1], _ptr(plan), n_real, n_rows, 1 if swiglu else 0, _ptr(out),
          1 if out.dtype == torch.float32 else 0, 1 if blocked else 0, _stream())
    return True


def moe_gather(a, row_pair, pairs_per_token: int, plan, n_real: int, out) -> None:
    """out[r] = a[row_pair[r] / pairs_per_token] for the rows the plan has in use."""
    if out.dtype != a.dtype or not out.is_contiguous():
        raise KernelError("moe_gather: one dtype, a contiguous output")
    f = _fn("moe.cu", "g2b_moe_gather",
            [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
    _call(f, _ptr(a), _code(a.dtype), _dense_rows(a, "a"), _ptr(row_pair), pairs_per_token, _ptr(plan), n_real,
          out.shape[0], a.shape[1], _ptr(out), _stream())


def moe_gemm_tc(a_rows, w, n_out: int, plan, n_real: int, max_tiles: int, swiglu: bool, out) -> bool:
    """``moe_gemm`` on the tcgen05 kernel: ``a_rows`` [rows, K] bfloat16, gathered in the plan's order;
    ``w`` [E, n_out (x2, blocked, with ``swiglu``), K]; out float32 [rows, n_out], or bfloat16 with
    ``swiglu``.  False when the sizes do not fit the kernel."""
    if a_rows.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    return (_bf16 or _bf16_mod()).gemm_tc_grouped(a_rows, w, n_out, plan, n_real, max_tiles, swiglu, out)


def moe_combine(rows32, pair_row, weight, x_self32, top: int, out32, accumulate: bool = False) -> None:
    """out[t] = sum_j weight[t, j] * (rows32[pair_row[t, j]], or x_self32[t] where the pair has no row);
    ``accumulate``: added to ``out32`` instead of stored."""
    f = _fn("moe.cu", "g2b_moe_combine", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int,
                                          c_void_p])
    _call(f, _ptr(rows32), _ptr(pair_row), _ptr(weight), _ptr(x_self32), out32.shape[0], top, out32.shape[1],
          _ptr(out32), 1 if accumulate else 0, _stream())


def moe_combine_norm_add(rows32, pair_row, weight, x32, norm_w, eps: float, top: int, cast_out=None) -> bool:
    """``moe_combine`` whose sum is not stored: x += sum / sqrt(mean(sum^2) + eps) * norm_w, the experts
    without matrices reading x as it was, and the new x once more, rounded, into ``cast_out``.  False
    for rows of more than 4,096 entries (the caller then runs the two kernels one after the other)."""
    if x32.shape[1] > 4096:
        return False
    _need(x32, torch.float32, "stream")
    if norm_w is not None:
        _need(norm_w, torch.float32, "norm weight")
    f = _fn("moe.cu", "g2b_moe_combine_norm_add",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_void_p, c_int, c_void_p])
    _call(f, _ptr(rows32), _ptr(pair_row), _ptr(weight), _ptr(x32), _ptr(norm_w), eps, x32.shape[0], top,
          x32.shape[1], _ptr(cast_out), _code(cast_out.dtype) if cast_out is not None else F32, _stream())
    return True
