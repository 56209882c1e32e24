"""Python signatures of the CUDA kernels.

Each function checks what the kernel cannot check itself (device, dtype, contiguity,
sizes it refuses), passes raw pointers and the current CUDA stream through ctypes, and
raises on a launch error.  Nothing here computes anything and nothing falls back to
another implementation: tensors that are not on a CUDA device are an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from . import build

F32, BF16 = 0, 1
BLOCK_TOKENS = 64          # tokens of one cache block (TT_BLOCK_TOKENS in csrc/common.cuh)
MAX_HEAD_DIM = 256

STATUS_BAD_TOKEN = 1
STATUS_BAD_BLOCK = 2
STATUS_WAIT_EXPIRED = 4
STATUS_BAD_SHAPE = 8


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(t: torch.Tensor | None) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("thintensor_b200 kernels run on CUDA tensors only; got a tensor on " + str(t.device))
    return c_void_p(t.data_ptr())


def _stream() -> c_void_p:
    # the raw handle of torch's current stream on the current device (torch.cuda.current_stream()
    # builds a Stream object around the same number, at ten times the cost)
    return c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


_launches = 0


def launch_count() -> int:
    """How many of this library's kernels have been launched (or captured into a graph)
    by this process so far."""
    return _launches


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _launches
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code} at launch")
    _launches += kernels


def _need(t: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_functions: dict[str, object] = {}


class ClassTimer:
    """Device time per class of kernel, for looking at where a step's time goes: while one is
    active (``with api.timed_classes() as timer``) every call of an entry point of this library is
    bracketed by two CUDA events on the current stream, and ``timer.summary()`` adds the spans up
    by entry point and label (parts label their matrix products: ``attention.qkv``, ``ffn.down``
    ...).  The events keep a kernel from starting under the tail of the one before it, so the
    spans are those of kernels run one after another, like a profiler's: compare shares, and take
    a step's duration from an untimed run.  Not for use while a CUDA graph is being captured.
    The reference's counterpart brackets layers the same way (LayerProfileEvents,
    thinruntime/gpu_runtime.py:4770-4797, summed at :7464-7543)."""

    def __init__(self):
        self.spans: list[tuple[str, torch.cuda.Event, torch.cuda.Event]] = []

    def wrap(self, name: str, fn):
        def timed(*args):
            global _label
            key = name if _label is None else f"{name}[{_label}]"
            _label = None
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            code = fn(*args)
            stop.record()
            self.spans.append((key, start, stop))
            return code

        return timed

    def summary(self) -> dict[str, dict]:
        """class -> {"calls": n, "ms": total}; synchronises."""
        torch.cuda.synchronize()
        out: dict[str, dict] = {}
        for key, start, stop in self.spans:
            entry = out.setdefault(key, {"calls": 0, "ms": 0.0})
            entry["calls"] += 1
            entry["ms"] += start.elapsed_time(stop)
        return dict(sorted(out.items(), key=lambda item: -item[1]["ms"]))


_timer: ClassTimer | None = None
_label: str | None = None


def set_label(label: str) -> None:
    """Name the next kernel call for an active :class:`ClassTimer` (no effect otherwise)."""
    global _label
    if _timer is not None:
        _label = label


class timed_classes:
    """Context manager that switches a :class:`ClassTimer` on for the calls inside it."""

    def __enter__(self) -> ClassTimer:
        global _timer
        if _timer is not None:
            raise KernelError("a class timer is already active")
        _timer = ClassTimer()
        return _timer

    def __exit__(self, *exc) -> None:
        global _timer, _label
        _timer, _label = None, None


def _fn(lib: str, name: str, argtypes: list):
    """The C entry point ``name`` of library ``lib`` (built and loaded at first use), with its prototype set."""
    fn = _functions.get(name)
    if fn is None:
        fn = getattr(build.load(lib), name)
        fn.argtypes = argtypes
        fn.restype = c_int
        _functions[name] = fn
    if _timer is not None:
        return _timer.wrap(name, fn)
    return fn


# ------------------------------------------------------------------------- elementwise
def embed_gather(table: torch.Tensor, tokens: torch.Tensor, residual: torch.Tensor, scale: float, status: torch.Tensor) -> None:
    """residual[t] = table[tokens[t]] * scale, float32 out."""
    _need(tokens, torch.int32, "tokens")
    _need(residual, torch.float32, "residual")
    if not table.is_contiguous():
        raise KernelError("embedding table must be contiguous")
    n, hidden = tokens.numel(), table.shape[1]
    fn = _fn("elementwise", "tt_embed_gather", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p])
    _check(fn(_ptr(table), dtype_code(table.dtype), _ptr(tokens), _ptr(residual), n, hidden, table.shape[0], scale, _ptr(status), _stream()), "embed_gather")


def embed_position_gather(table: torch.Tensor, positions: torch.Tensor, tokens: torch.Tensor, cu: torch.Tensor, len_before: torch.Tensor,
                          sequences: int, residual: torch.Tensor, scale: float, status: torch.Tensor) -> None:
    """residual[t] = table[tokens[t]] * scale + positions[p] with p the position of packed token t in its sequence."""
    _need(tokens, torch.int32, "tokens")
    _need(residual, torch.float32, "residual")
    if not table.is_contiguous() or not positions.is_contiguous() or table.dtype != positions.dtype:
        raise KernelError("embedding tables must be contiguous and of one dtype")
    if positions.shape[1] != table.shape[1]:
        raise KernelError(f"the position table must have rows of {table.shape[1]} numbers, got {tuple(positions.shape)}")
    n, hidden = tokens.numel(), table.shape[1]
    fn = _fn("elementwise", "tt_embed_position_gather", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                                         c_int, c_int, c_float, c_void_p, c_void_p])
    _check(fn(_ptr(table), _ptr(positions), dtype_code(table.dtype), _ptr(tokens), _ptr(cu), _ptr(len_before), sequences, _ptr(residual), n,
              hidden, table.shape[0], positions.shape[0], scale, _ptr(status), _stream()), "embed_position_gather")


def embed_pair_gather(table: torch.Tensor, pair_table: torch.Tensor, tokens: torch.Tensor, cu: torch.Tensor, slots: torch.Tensor,
                      sequences: int, last_token: torch.Tensor, residual: torch.Tensor, buckets: int, mul_prev: int, mul_cur: int,
                      scale: float, status: torch.Tensor) -> None:
    """residual[t] = table[tokens[t]] * scale + pair_table[(previous * mul_prev + tokens[t] * mul_cur) % buckets], and row
    ``buckets`` of ``pair_table`` for a sequence's first token.  ``last_token`` (int32 ``[slots]``, last token plus one, zero for a
    sequence without tokens) gives the token before the step's first one and is moved on to the step's last."""
    _need(tokens, torch.int32, "tokens")
    _need(residual, torch.float32, "residual")
    _need(last_token, torch.int32, "the sequences' last tokens")
    if not table.is_contiguous() or not pair_table.is_contiguous() or table.dtype != pair_table.dtype:
        raise KernelError("embedding tables must be contiguous and of one dtype")
    if pair_table.shape[0] != buckets + 1 or pair_table.shape[1] != table.shape[1]:
        raise KernelError(f"the pair table must be [{buckets + 1}, {table.shape[1]}], got {tuple(pair_table.shape)}")
    n, hidden = tokens.numel(), table.shape[1]
    fn = _fn("elementwise", "tt_embed_pair_gather", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                     c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_float, c_void_p, c_void_p])
    _check(fn(_ptr(table), _ptr(pair_table), dtype_code(table.dtype), _ptr(tokens), _ptr(cu), _ptr(slots), sequences, _ptr(last_token),
              _ptr(residual), n, hidden, table.shape[0], buckets, mul_prev, mul_cur, scale, _ptr(status), _stream()), "embed_pair_gather")


def token_shift(x: torch.Tensor, mix: torch.Tensor, state: torch.Tensor, out: torch.Tensor, cu: torch.Tensor, slots: torch.Tensor,
                sequences: int) -> None:
    """out[t] = x[t] + (x[t - 1] - x[t]) * mix within each sequence; the row before a step's first one is ``state[slot]``
    (float32 ``[slots, hidden]``, zero for a new sequence), which is moved on to the step's last row."""
    _need(mix, torch.float32, "shift weights")
    _need(state, torch.float32, "shift state")
    if x.dtype != out.dtype or x.shape != out.shape or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("token_shift: input and output must be contiguous and alike")
    tokens, hidden = x.shape
    if mix.numel() != hidden or state.shape[1] != hidden:
        raise KernelError("token_shift: weights or state do not fit the width")
    fn = _fn("elementwise", "tt_token_shift", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(x), dtype_code(x.dtype), _ptr(mix), _ptr(state), _ptr(out), _ptr(cu), _ptr(slots), sequences, tokens, hidden, _stream()),
           "token_shift")


def add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: torch.Tensor | None = None, weight_offset: float = 0.0) -> None:
    """residual += sum(delta over its first axis); out = rmsnorm(residual) * weight.
    With ``rows`` (int32), out[i] comes from residual row rows[i] and residual is left
    as it was."""
    _need(residual, torch.float32, "residual")
    _need(weight, torch.float32, "norm weight")
    if not out.is_contiguous():
        raise KernelError("norm output must be contiguous")
    hidden = residual.shape[-1]
    splits, stride = 0, 0
    if delta is not None:
        _need(delta, torch.float32, "delta")
        splits = delta.shape[0]
        stride = delta.stride(0)
    n_rows = rows.numel() if rows is not None else residual.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows")
    fn = _fn("elementwise", "tt_add_rmsnorm", [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_float, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(residual), _ptr(delta), splits, stride, _ptr(weight), weight_offset, eps, _ptr(out), dtype_code(out.dtype), _ptr(rows), n_rows, hidden, _stream()), "add_rmsnorm")


def add_rmsnorm_chain(residual: torch.Tensor, delta: torch.Tensor | None, post_weight: torch.Tensor | None, post_offset: float, post_eps: float,
                      results: torch.Tensor | None, index: int, depth_weights: torch.Tensor | None, weight: torch.Tensor, weight_offset: float,
                      eps: float, out: torch.Tensor, rows: torch.Tensor | None = None) -> None:
    """:func:`add_rmsnorm` with two more steps on the way.  The summed delta is first normalised,
    ``v * rsqrt(mean(v^2) + post_eps) * (post_weight + post_offset)`` (``post_weight`` None: added as it is).  After the
    addition the stream is kept as ``results[index]`` (float32 ``[count, tokens, hidden]``) and, with ``depth_weights``
    (float32, at least ``index + 1`` numbers), replaced by ``sum(depth_weights[j] * results[j] for j <= index)``.  With
    ``rows`` nothing but ``out`` is written."""
    _need(residual, torch.float32, "residual")
    _need(weight, torch.float32, "norm weight")
    if not out.is_contiguous():
        raise KernelError("norm output must be contiguous")
    hidden = residual.shape[-1]
    splits, stride = 0, 0
    if delta is not None:
        _need(delta, torch.float32, "delta")
        splits, stride = delta.shape[0], delta.stride(0)
    if post_weight is not None:
        _need(post_weight, torch.float32, "norm weight of the delta")
        if delta is None:
            raise KernelError("a norm of the delta needs a delta")
    result_stride = 0
    if results is not None:
        _need(results, torch.float32, "results")
        if results.dim() != 3 or tuple(results.shape[1:]) != tuple(residual.shape) or not 0 <= index < results.shape[0]:
            raise KernelError(f"results must be [count > {index}, {residual.shape[0]}, {hidden}], got {tuple(results.shape)}")
        result_stride = results.stride(0)
    if depth_weights is not None:
        _need(depth_weights, torch.float32, "depth weights")
        if results is None or depth_weights.numel() < index + 1:
            raise KernelError(f"mixing results 0..{index} needs the results and {index + 1} weights")
    n_rows = rows.numel() if rows is not None else residual.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows")
    fn = _fn("elementwise", "tt_add_rmsnorm_chain", [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_float, c_float, c_void_p, c_longlong, c_int,
                                                     c_void_p, c_void_p, c_float, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(residual), _ptr(delta), splits, stride, _ptr(post_weight), post_offset, post_eps, _ptr(results), result_stride, index,
              _ptr(depth_weights), _ptr(weight), weight_offset, eps, _ptr(out), dtype_code(out.dtype), _ptr(rows), n_rows, hidden, _stream()),
           "add_rmsnorm_chain")


def add_layernorm(residual: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, bias: torch.Tensor | None, eps: float,
                  out: torch.Tensor, rows: torch.Tensor | None = None) -> None:
    """residual += sum(delta over its first axis); out = (x - mean) / sqrt(var + eps) * weight (+ bias), the
    variance being the mean squared deviation.  ``rows`` as for :func:`add_rmsnorm`."""
    _need(residual, torch.float32, "residual")
    _need(weight, torch.float32, "norm weight")
    if bias is not None:
        _need(bias, torch.float32, "norm bias")
    if not out.is_contiguous():
        raise KernelError("norm output must be contiguous")
    hidden = residual.shape[-1]
    splits, stride = 0, 0
    if delta is not None:
        _need(delta, torch.float32, "delta")
        splits, stride = delta.shape[0], delta.stride(0)
    n_rows = rows.numel() if rows is not None else residual.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows")
    fn = _fn("elementwise", "tt_add_layernorm", [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(residual), _ptr(delta), splits, stride, _ptr(weight), _ptr(bias), eps, _ptr(out), dtype_code(out.dtype), _ptr(rows), n_rows, hidden, _stream()), "add_layernorm")


def qk_norm_rope_append(proj: torch.Tensor, q_norm: torch.Tensor | None, k_norm: torch.Tensor | None, norm_eps: float,
                        inv_freq: torch.Tensor, rotary_dim: int, interleaved: bool, attention_scaling: float, q_out: torch.Tensor,
                        k_pool: torch.Tensor | None, v_pool: torch.Tensor | None, table: torch.Tensor, cu: torch.Tensor,
                        len_before: torch.Tensor, sequences: int, n_tokens: int, heads: int, kv_heads: int, head_dim: int,
                        value_dim: int, status: torch.Tensor, cos_sin: torch.Tensor | None = None,
                        where: torch.Tensor | None = None, unit_norm: bool = False, q_gain: tuple[float, int] | None = None,
                        value_from_keys: bool = False) -> None:
    """The general form of :func:`rope_append`: float32 partial sums ``proj`` [splits, tokens, cols] hold q heads, then k
    heads (``head_dim`` numbers each), then v heads (``value_dim`` each).  q and k are normalised per head (x / rms(x) *
    weight; ``q_norm`` / ``k_norm`` float32 [head_dim] or None), then their first ``rotary_dim`` numbers are rotated, in
    neighbouring pairs (``interleaved``) or in halves; q goes to ``q_out``, k and v to the block pools.  Without pools
    the projection holds queries only.  ``cos_sin`` and ``where``: the step's :func:`rope_table` for this layer's
    frequencies, looked up instead of computing positions, cosines and sines per head.  ``unit_norm``: q and k are
    normalised without a weight.  ``q_gain`` = (coef, every): queries at position p are multiplied by
    ``1 + coef * ln(floor((p + 1) / every) + 1)``.  ``value_from_keys``: the projection has no v heads; a value head is its
    key head before the norm."""
    proj_ptr, proj_splits, proj_stride, proj_row, _ = _projection_view(proj)     # may be the leading columns of a wider projection
    _need(inv_freq, torch.float32, "inv_freq")
    write = k_pool is not None
    if value_from_keys and value_dim != head_dim:
        raise KernelError("values that are the keys have the keys' size")
    if q_gain is not None and int(q_gain[1]) < 1:
        raise KernelError("the query gain's period must be at least one position")
    cols = heads * head_dim + (kv_heads * (head_dim + (0 if value_from_keys else value_dim)) if write else 0)
    if proj.shape[-1] != cols:
        raise KernelError(f"the projection has {proj.shape[-1]} columns, expected {cols}")
    for norm in (q_norm, k_norm):
        if norm is not None:
            _need(norm, torch.float32, "query/key norm weight")
            if norm.numel() != head_dim:
                raise KernelError(f"a query/key norm weight must have {head_dim} numbers")
    if write and (k_pool.dtype != q_out.dtype or v_pool.dtype != q_out.dtype):
        raise KernelError("cache pools and activations must share a dtype")
    if rotary_dim and inv_freq.numel() < rotary_dim // 2:
        raise KernelError("the rotary table is shorter than half the rotary part")
    if (cos_sin is None) != (where is None):
        raise KernelError("the step's rope table comes as both of cos_sin and where, or neither")
    if cos_sin is not None:
        _need(cos_sin, torch.float32, "cos/sin table")
        _need(where, torch.int32, "token positions")
        if tuple(cos_sin.shape) != (n_tokens, rotary_dim // 2, 2) or tuple(where.shape) != (n_tokens, 2):
            raise KernelError("the rope table does not fit the step")
    fn = _fn("elementwise", "tt_qk_norm_rope_append", [c_void_p, c_int, c_longlong, c_int, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int,
                                                       c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                                       c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_int,
                                                       c_int, c_void_p, c_void_p])
    _check(fn(proj_ptr, proj_splits, proj_stride, proj_row, _ptr(q_norm), _ptr(k_norm), norm_eps, _ptr(inv_freq), rotary_dim,
              1 if interleaved else 0, attention_scaling, _ptr(q_out), _ptr(k_pool), _ptr(v_pool), dtype_code(q_out.dtype), _ptr(table),
              table.shape[1], k_pool.shape[0] if write else 0, _ptr(cu), _ptr(len_before), sequences, n_tokens, heads, kv_heads, head_dim,
              value_dim, 1 if write else 0, _ptr(cos_sin), _ptr(where), 1 if unit_norm else 0, 0.0 if q_gain is None else float(q_gain[0]),
              0 if q_gain is None else int(q_gain[1]), 1 if value_from_keys else 0, _ptr(status), _stream()), "qk_norm_rope_append")


def rope_append(qkv: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int, attention_scaling: float, q_out: torch.Tensor,
                k_pool: torch.Tensor | None, v_pool: torch.Tensor | None, table: torch.Tensor | None, cu: torch.Tensor,
                len_before: torch.Tensor, sequences: int, n_tokens: int, heads: int, kv_heads: int, head_dim: int,
                status: torch.Tensor) -> None:
    """Rotate q and k of float32 partial sums ``qkv`` [splits, tokens, cols], write q in
    the activation dtype and append k and v to the block pools.  Without pools the
    projection holds queries only."""
    _need(qkv, torch.float32, "qkv")
    _need(inv_freq, torch.float32, "inv_freq")
    write = k_pool is not None
    cols = heads * head_dim + (2 * kv_heads * head_dim if write else 0)
    if qkv.shape[-1] != cols:
        raise KernelError(f"qkv has {qkv.shape[-1]} columns, expected {cols}")
    if write and (k_pool.dtype != q_out.dtype or v_pool.dtype != q_out.dtype):
        raise KernelError("cache pools and activations must share a dtype")
    fn = _fn("elementwise", "tt_rope_append", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int,
                                               c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(qkv), qkv.shape[0], qkv.stride(0), _ptr(inv_freq), rotary_dim, attention_scaling, _ptr(q_out), _ptr(k_pool), _ptr(v_pool),
              dtype_code(q_out.dtype), _ptr(table), table.shape[1] if table is not None else 0,
              k_pool.shape[0] if write else 0, _ptr(cu), _ptr(len_before), sequences, n_tokens, heads, kv_heads, head_dim,
              1 if write else 0, _ptr(status), _stream()), "rope_append")


def rope_table(inv_freq: torch.Tensor, rotary_dim: int, cu: torch.Tensor, len_before: torch.Tensor, sequences: int, n_tokens: int,
               cos_sin: torch.Tensor, where: torch.Tensor) -> None:
    """What the rotations of all layers of a step share: ``where[t] = (position, sequence)`` of packed token t
    (int32 [tokens, 2]) and ``cos_sin[t, i] = (cos, sin)(inv_freq[i] * position)`` (float32 [tokens, rotary_dim / 2, 2])."""
    _need(inv_freq, torch.float32, "inv_freq")
    _need(cos_sin, torch.float32, "cos/sin table")
    _need(where, torch.int32, "token positions")
    half = rotary_dim // 2
    if tuple(cos_sin.shape) != (n_tokens, half, 2) or tuple(where.shape) != (n_tokens, 2) or inv_freq.numel() < half:
        raise KernelError(f"rope_table: cos_sin must be [{n_tokens}, {half}, 2] and where [{n_tokens}, 2]")
    fn = _fn("elementwise", "tt_rope_table", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(inv_freq), half, _ptr(cu), _ptr(len_before), sequences, n_tokens, _ptr(cos_sin), _ptr(where), _stream()), "rope_table")


GATE_ACTIVATIONS = {"silu": 0, "relu": 1, "gelu_tanh": 2}


def swiglu(gate_up: torch.Tensor, act: torch.Tensor, activation: str = "silu") -> None:
    """act = f(gate) * up from float32 partial sums [splits, tokens, 2 * inter]; f is silu, relu or the
    tanh form of gelu."""
    _need(gate_up, torch.float32, "gate_up")
    if activation not in GATE_ACTIVATIONS:
        raise KernelError(f"gate activation {activation!r} is not one of {sorted(GATE_ACTIVATIONS)}")
    inter = gate_up.shape[-1] // 2
    fn = _fn("elementwise", "tt_swiglu", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(gate_up), gate_up.shape[0], gate_up.stride(0), _ptr(act), dtype_code(act.dtype), gate_up.shape[1], inter,
              GATE_ACTIVATIONS[activation], _stream()), "swiglu")


UNARY_ACTIVATIONS = {**GATE_ACTIVATIONS, "xielu": 3, "gelu": 4}      # gelu: the exact one, with erf


def activation(x: torch.Tensor, act: torch.Tensor, activation: str = "gelu_tanh", a: float = 0.0, c: float = 0.0) -> None:
    """act = f(sum of the float32 slices ``x`` [splits, tokens, inter]) in the activation dtype.  ``xielu`` takes the two
    numbers a = softplus(p) and c = 1 / 2 + softplus(q): ``a z^2 + z / 2`` for z > 0, ``c (exp(z) - 1 - z) + z / 2`` otherwise."""
    _need(x, torch.float32, "the activation's input")
    if x.dim() != 3 or tuple(act.shape) != tuple(x.shape[1:]) or not act.is_contiguous():
        raise KernelError("activation: the output must be contiguous [tokens, inter] for an input [splits, tokens, inter]")
    fn = _fn("elementwise", "tt_activation", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_longlong, c_int, c_float, c_float, c_void_p])
    _check(fn(_ptr(x), x.shape[0], x.stride(0), _ptr(act), dtype_code(act.dtype), act.numel(), UNARY_ACTIVATIONS[activation], a, c, _stream()),
           "activation")


def copy_int32(dst: torch.Tensor, src: torch.Tensor, extra: torch.Tensor | None = None) -> None:
    """dst[:n] = src for small int32 vectors; either side may be pinned host memory.  With ``extra``
    (one int32 on the device, the status word say) ``dst`` has n + 1 entries and dst[n] = extra[0]."""
    for t, name in ((dst, "dst"), (src, "src")):
        if t.dtype != torch.int32 or not t.is_contiguous() or not (t.is_cuda or t.is_pinned()):
            raise KernelError(f"copy_int32: {name} must be contiguous int32 on the device or in pinned host memory")
    if dst.numel() != src.numel() + (1 if extra is not None else 0):
        raise KernelError("copy_int32: sizes differ")
    if extra is not None and (extra.dtype != torch.int32 or extra.numel() != 1 or not extra.is_cuda):
        raise KernelError("copy_int32: the extra word must be one int32 on the device")
    fn = _fn("elementwise", "tt_copy_int32", [c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    _check(fn(c_void_p(dst.data_ptr()), c_void_p(src.data_ptr()), src.numel(), _ptr(extra), _stream()), "copy_int32")


def advance_lengths(lengths: torch.Tensor, cu: torch.Tensor, sequences: int, counters: torch.Tensor | None = None) -> None:
    """lengths[b] += cu[b + 1] - cu[b] after a step; ``counters`` (int32, one per sequence), if given, go up by one."""
    if counters is not None:
        _need(counters, torch.int32, "step counters")
    fn = _fn("elementwise", "tt_advance_lengths", [c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(lengths), _ptr(cu), _ptr(counters), sequences, _stream()), "advance_lengths")


# --------------------------------------------------------------------------- attention
def check_head_dim(head_dim: int) -> None:
    if head_dim <= 0 or head_dim > MAX_HEAD_DIM:
        raise KernelError(f"attention kernels take head sizes up to {MAX_HEAD_DIM}, not {head_dim}")


def attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor, cu: torch.Tensor,
              len_before: torch.Tensor, sequences: int, n_tokens: int, heads: int, kv_heads: int, head_dim: int,
              scale: float, window: int, splits: int, out: torch.Tensor, part_acc: torch.Tensor | None,
              part_ml: torch.Tensor | None, status: torch.Tensor, value_dim: int | None = None,
              sinks: torch.Tensor | None = None, softcap: float = 0.0, slopes: torch.Tensor | None = None,
              gate: torch.Tensor | None = None, gate_per_head: bool = False) -> None:
    """Exact causal attention of ``n_tokens`` packed query tokens over the block cache.  ``value_dim``: the size of a
    value head where it differs from the keys'.  ``sinks`` (float32, one per query head): a term exp(sink) in the
    softmax denominator that has no key and no value and is not scaled.  ``softcap`` > 0: a scaled score s becomes
    ``softcap * tanh(s / softcap)``.  ``slopes`` (float32, one per query head): ``slope_h * (i - j)`` is taken off the score of
    query position i and key position j.  ``gate``: float32 partial sums ``[slices, tokens, heads * value_dim]`` (with
    ``gate_per_head``: ``[slices, tokens, heads]``), possibly a range of a wider projection's columns; the output is
    multiplied by their sigmoid."""
    check_head_dim(head_dim)
    value_dim = head_dim if value_dim is None else int(value_dim)
    check_head_dim(value_dim)
    _check_sinks(sinks, heads)
    if heads % kv_heads:
        raise KernelError(f"{heads} query heads are not a multiple of {kv_heads} key/value heads")
    if not (q.dtype == k_pool.dtype == v_pool.dtype == out.dtype):
        raise KernelError("queries, cache and output must share a dtype")
    if slopes is not None:
        _need(slopes, torch.float32, "slopes")
        if slopes.numel() != heads:
            raise KernelError(f"a slope per query head: {heads} numbers, got {slopes.numel()}")
    g_ptr, g_splits, g_stride, g_row = c_void_p(0), 0, 0, 0
    if gate is not None:
        g_ptr, g_splits, g_stride, g_row, g_cols = _projection_view(gate)
        if g_cols != (heads if gate_per_head else heads * value_dim) or gate.shape[1] != n_tokens:
            raise KernelError("attention: the gate does not fit the heads")
    fn = _fn("attention", "tt_attention", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                                           c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_float, c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p])
    _check(fn(_ptr(q), _ptr(k_pool), _ptr(v_pool), dtype_code(q.dtype), _ptr(table), table.shape[1], k_pool.shape[0], _ptr(cu),
              _ptr(len_before), sequences, n_tokens, heads, kv_heads, head_dim, value_dim, scale, _ptr(sinks), window, splits, _ptr(out),
              _ptr(part_acc), _ptr(part_ml), _ptr(status), float(softcap or 0.0), _ptr(slopes), g_ptr, g_splits, g_stride, g_row,
              1 if gate_per_head else 0, _stream()), "attention", 2 if splits > 1 else 1)


def differential_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor, cu: torch.Tensor,
                           len_before: torch.Tensor, sequences: int, n_tokens: int, heads: int, kv_heads: int, dim: int, value_dim: int,
                           scale: float, lam: float, gain: float, eps: float, splits: int, out: torch.Tensor,
                           part_acc: torch.Tensor | None, part_ml: torch.Tensor | None, status: torch.Tensor) -> None:
    """Causal differential attention over the block cache: query rows ``[tokens, heads, 2 * dim]`` and cached key rows of
    ``2 * dim`` numbers hold two maps; ``out[t, h] = norm(a1 - lam * a2) * gain`` with a1, a2 the two maps' softmax
    attentions over the same values (``value_dim`` numbers a head) and norm the division by ``sqrt(mean(o^2) + eps)``.
    ``part_acc`` / ``part_ml`` (float32, ``tokens * heads * splits * 2 * value_dim`` and ``... * 4`` numbers) for splits > 1."""
    if k_pool.dtype != q.dtype or v_pool.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("queries, cache and output must share a dtype")
    if k_pool.shape[-1] != 2 * dim or q.shape[-1] != heads * 2 * dim:
        raise KernelError("differential attention: rows of queries and keys hold two maps of dim numbers")
    if splits > 1:
        _need(part_acc, torch.float32, "partial accumulators")
        _need(part_ml, torch.float32, "partial maxima and sums")
        if part_acc.numel() < n_tokens * heads * splits * 2 * value_dim or part_ml.numel() < n_tokens * heads * splits * 4:
            raise KernelError("differential attention: scratch for the slices is too small")
    fn = _fn("attention_forms", "tt_differential_attention", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                                                              c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_float, c_int, c_void_p,
                                                              c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(q), _ptr(k_pool), _ptr(v_pool), dtype_code(q.dtype), _ptr(table), table.shape[1], k_pool.shape[0], _ptr(cu), _ptr(len_before),
              sequences, n_tokens, heads, kv_heads, dim, value_dim, scale, lam, gain, eps, splits, _ptr(out), _ptr(part_acc), _ptr(part_ml),
              _ptr(status), _stream()), "differential_attention", 2 if splits > 1 else 1)


def attention_forms_on_tensor_cores(dtype: torch.dtype, differential: bool, heads: int, kv_heads: int, dim: int, value_dim: int) -> bool:
    """Whether differential attention (``dim`` numbers a map) or window attention with pooled blocks (``value_dim == dim``)
    runs on tensor cores at these sizes: bfloat16, and a size the kernels are built for; its parallel unit is then a
    (sequence, key/value head) pair and not a (token, query head) row."""
    if dtype != torch.bfloat16:
        return False
    fn = _fn("attention_forms", "tt_attention_forms_on_tensor_cores", [c_int, c_int, c_int, c_int, c_int])
    return bool(fn(1 if differential else 0, heads, kv_heads, dim, value_dim))


def pool_blocks(k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor, mean_k: torch.Tensor, mean_v: torch.Tensor,
                mean_table: torch.Tensor, cu: torch.Tensor, len_before: torch.Tensor, sequences: int, most_blocks: int, kv_heads: int,
                head_dim: int, value_dim: int, every: int, status: torch.Tensor) -> None:
    """For every block of ``every`` tokens that this step completes (tokens ``n * every .. n * every + every - 1`` with the last
    one among the step's), the mean of the block's cached keys and the mean of its cached values, written as entry n of
    the coarser cache ``mean_k`` / ``mean_v`` (laid out like the token pools, addressed through ``mean_table``).
    ``most_blocks`` bounds the blocks one sequence can complete in the step."""
    if mean_k.dtype != k_pool.dtype or mean_v.dtype != k_pool.dtype:
        raise KernelError("the token cache and the coarser cache must share a dtype")
    fn = _fn("attention_forms", "tt_pool_blocks", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                                   c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _check(fn(_ptr(k_pool), _ptr(v_pool), dtype_code(k_pool.dtype), _ptr(table), table.shape[1], k_pool.shape[0], _ptr(mean_k), _ptr(mean_v),
              _ptr(mean_table), mean_table.shape[1], mean_k.shape[0], _ptr(cu), _ptr(len_before), sequences, most_blocks, kv_heads, head_dim,
              value_dim, every, _ptr(status), _stream()), "pool_blocks")


def pooled_window_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor, mean_k: torch.Tensor,
                            mean_v: torch.Tensor, mean_table: torch.Tensor, every: int, cu: torch.Tensor, len_before: torch.Tensor,
                            sequences: int, n_tokens: int, heads: int, kv_heads: int, head_dim: int, scale: float, cap: float, window: int,
                            splits: int, out: torch.Tensor, part_acc: torch.Tensor | None, part_ml: torch.Tensor | None,
                            status: torch.Tensor) -> None:
    """Attention of position i over the keys ``i - window < j <= i`` and, in the same softmax, over entry n of the coarser
    cache for every block of ``every`` tokens with ``n * every + every - 1 <= i - window``; ``cap`` > 0 caps the scores,
    ``cap * tanh(s / cap)``.  Values have the keys' size."""
    if k_pool.dtype != q.dtype or v_pool.dtype != q.dtype or out.dtype != q.dtype or mean_k.dtype != q.dtype or mean_v.dtype != q.dtype:
        raise KernelError("queries, caches and output must share a dtype")
    if splits > 1:
        _need(part_acc, torch.float32, "partial accumulators")
        _need(part_ml, torch.float32, "partial maxima and sums")
        if part_acc.numel() < n_tokens * heads * splits * head_dim or part_ml.numel() < n_tokens * heads * splits * 2:
            raise KernelError("pooled window attention: scratch for the slices is too small")
    fn = _fn("attention_forms", "tt_pooled_window_attention", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                                               c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                               c_float, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(q), _ptr(k_pool), _ptr(v_pool), dtype_code(q.dtype), _ptr(table), table.shape[1], k_pool.shape[0], _ptr(mean_k), _ptr(mean_v),
              _ptr(mean_table), mean_table.shape[1], mean_k.shape[0], every, _ptr(cu), _ptr(len_before), sequences, n_tokens, heads, kv_heads,
              head_dim, scale, cap, window, splits, _ptr(out), _ptr(part_acc), _ptr(part_ml), _ptr(status), _stream()),
           "pooled_window_attention", 2 if splits > 1 else 1)


def _attention_launches(splits: int, decode: bool, tickets: bool = False) -> int:
    """Kernels one call launches: the decode kernel combines up to 8 slices itself (a thread-block
    cluster) and, given tickets, any number; otherwise more slices need the merge kernel."""
    return 1 if splits == 1 or (decode and (splits <= 8 or tickets)) else 2


def _check_sinks(sinks: torch.Tensor | None, heads: int) -> None:
    """``sinks``: float32, one per query head; exp(sink) joins the softmax denominator with no key, no value and no scale."""
    if sinks is not None:
        _need(sinks, torch.float32, "sinks")
        if sinks.numel() != heads:
            raise KernelError(f"attention with {heads} query heads needs {heads} sinks, got {sinks.numel()}")


def _check_tickets(tickets: torch.Tensor | None, sequences: int, kv_heads: int) -> None:
    if tickets is not None:
        _need(tickets, torch.int32, "tickets")
        if tickets.numel() < sequences * kv_heads:
            raise KernelError(f"decode attention needs {sequences * kv_heads} tickets, got {tickets.numel()}")


def attention_mma_supports(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether the tensor-core attention kernel takes these sizes (bfloat16, head size 32,
    64, 96 or 128, at most 16 query heads per key/value head)."""
    return dtype == torch.bfloat16 and head_dim in (32, 64, 96, 128) and heads % kv_heads == 0 and heads // kv_heads <= 16


def attention_mma(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor, cu: torch.Tensor,
                  len_before: torch.Tensor, sequences: int, n_tokens: int, heads: int, kv_heads: int, head_dim: int,
                  scale: float, window: int, splits: int, out: torch.Tensor, part_acc: torch.Tensor | None,
                  part_ml: torch.Tensor | None, status: torch.Tensor, one_token_each: bool = False,
                  tickets: torch.Tensor | None = None, sinks: torch.Tensor | None = None, softcap: float = 0.0,
                  slopes: torch.Tensor | None = None) -> None:
    """Causal attention of packed bfloat16 query tokens over the block cache on tensor cores.
    ``one_token_each`` (decoding): the warps of a CTA share a sequence's tile and split its keys.
    ``softcap`` and ``slopes`` (decoding only): see :func:`attention`.
    ``tickets`` (decoding; int32, one per sequence and key/value head, zero before the call and after it): with
    more slices than a cluster combines, the CTA that finishes last combines them and no second kernel runs."""
    if not attention_mma_supports(q.dtype, heads, kv_heads, head_dim):
        raise KernelError(f"the tensor-core attention kernel does not take {q.dtype}, {heads}/{kv_heads} heads of size {head_dim}")
    if not (k_pool.dtype == v_pool.dtype == out.dtype == torch.bfloat16):
        raise KernelError("queries, cache and output must all be bfloat16")
    if one_token_each and n_tokens != sequences:
        raise KernelError("one_token_each needs exactly one token per sequence")
    tickets = tickets if one_token_each else None
    _check_tickets(tickets, sequences, kv_heads)
    _check_sinks(sinks, heads)
    if sinks is not None and not one_token_each:
        raise KernelError("the tensor-core kernel of this file takes sinks only when decoding; prompts with sinks run attention_tcgen05 or attention")
    shaped = bool(softcap) or slopes is not None
    if shaped and not one_token_each:
        raise KernelError("the tensor-core kernel of this file shapes scores only when decoding; such prompts run attention_tcgen05 or attention")
    if slopes is not None:
        _need(slopes, torch.float32, "slopes")
        if slopes.numel() != heads:
            raise KernelError(f"a slope per query head: {heads} numbers, got {slopes.numel()}")
    if shaped:
        tickets = None                  # the shaped instances combine slices in a cluster or through the merge kernel
    fn = _fn("attention_mma", "tt_attention_mma", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                                                   c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                   c_float, c_void_p, c_void_p])
    _check(fn(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(table), table.shape[1], k_pool.shape[0], _ptr(cu), _ptr(len_before), sequences,
              n_tokens, heads, kv_heads, head_dim, scale, window, splits, sequences if one_token_each else 0, _ptr(out), _ptr(part_acc),
              _ptr(part_ml), _ptr(tickets), _ptr(status), _ptr(sinks), float(softcap or 0.0), _ptr(slopes),
              _stream()), "attention_mma", _attention_launches(splits, one_token_each, tickets is not None))


def attention_mma_failure_drill(wait_limit_ns: int, undelivered_bytes: int) -> None:
    """For tests of the failure path, never for serving.  ``wait_limit_ns``: the limit of the bounded waits in the
    tensor-core decode attention (0 restores the default of two seconds).  ``undelivered_bytes``: from now on the first
    stage of every warp expects that many bytes more than its copies bring (0 restores normal operation), so its barrier
    never completes; the kernel must then raise ``STATUS_WAIT_EXPIRED`` and return."""
    lib = build.load("attention_mma")
    lib.tt_attention_mma_failure_drill.argtypes = [c_ulonglong, c_int]
    lib.tt_attention_mma_failure_drill.restype = c_int
    code = lib.tt_attention_mma_failure_drill(int(wait_limit_ns), int(undelivered_bytes))
    if code != 0:
        raise KernelError(f"the decode attention's failure drill could not be set: CUDA error {code}")


def attention_decode_rope_supports(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int, rotary_dim: int) -> bool:
    """Whether decoding may rotate q and k and write the cache inside the attention kernel
    (bfloat16, head size 64 rotated whole, at most 16 query heads per key/value head)."""
    return attention_mma_supports(dtype, heads, kv_heads, head_dim) and head_dim == 64 and rotary_dim == head_dim


def attention_decode_rope(qkv: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int, attention_scaling: float, write_cache: bool,
                          k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor, len_before: torch.Tensor,
                          sequences: int, heads: int, kv_heads: int, head_dim: int, scale: float, window: int, splits: int,
                          out: torch.Tensor, part_acc: torch.Tensor | None, part_ml: torch.Tensor | None,
                          status: torch.Tensor, tickets: torch.Tensor | None = None) -> None:
    """One decode step of attention straight from the float32 partial sums ``qkv``
    [slices, sequences, cols] of the qkv product: q and k are rotated, k and v are written to
    the cache (``write_cache``; else ``qkv`` holds queries only), then every sequence's token
    attends over its cache: one launch where rope_append and attention_mma would be two."""
    _need(qkv, torch.float32, "qkv")
    _need(inv_freq, torch.float32, "inv_freq")
    if not attention_decode_rope_supports(out.dtype, heads, kv_heads, head_dim, rotary_dim):
        raise KernelError(f"the fused decode attention does not take {out.dtype}, {heads}/{kv_heads} heads of size {head_dim}, rotary part {rotary_dim}")
    if not (k_pool.dtype == v_pool.dtype == torch.bfloat16):
        raise KernelError("cache and output must be bfloat16")
    cols = heads * head_dim + (2 * kv_heads * head_dim if write_cache else 0)
    if qkv.shape[-1] != cols or qkv.shape[1] != sequences:
        raise KernelError(f"qkv is {tuple(qkv.shape)}, expected [slices, {sequences}, {cols}]")
    _check_tickets(tickets, sequences, kv_heads)
    fn = _fn("attention_mma", "tt_attention_decode_rope", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_float, c_int, c_void_p, c_void_p,
                                                           c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                                           c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(qkv), qkv.shape[0], qkv.stride(0), _ptr(inv_freq), rotary_dim, attention_scaling, 1 if write_cache else 0, _ptr(k_pool),
              _ptr(v_pool), _ptr(table), table.shape[1], k_pool.shape[0], _ptr(len_before), sequences, heads, kv_heads, head_dim, scale,
              window, splits, _ptr(out), _ptr(part_acc), _ptr(part_ml), _ptr(tickets), _ptr(status), _stream()), "attention_decode_rope",
           _attention_launches(splits, True, tickets is not None))


def attention_tcgen05_supports(dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether the tcgen05 prompt attention takes these sizes (bfloat16, head size 64 or 128,
    at most 16 query heads per key/value head)."""
    return dtype == torch.bfloat16 and head_dim in (64, 128) and heads % kv_heads == 0 and heads // kv_heads <= 16


def attention_tcgen05(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor, cu: torch.Tensor,
                      len_before: torch.Tensor, sequences: int, n_tokens: int, heads: int, kv_heads: int, head_dim: int,
                      scale: float, window: int, out: torch.Tensor, status: torch.Tensor, sinks: torch.Tensor | None = None,
                      softcap: float = 0.0, slopes: torch.Tensor | None = None, gate: torch.Tensor | None = None,
                      gate_per_head: bool = False) -> None:
    """Causal attention of packed bfloat16 prompts over the block cache with both products on
    the tcgen05 tensor cores.  ``sinks``, ``softcap``, ``slopes``, ``gate``: see :func:`attention`."""
    _check_sinks(sinks, heads)
    if slopes is not None:
        _need(slopes, torch.float32, "slopes")
        if slopes.numel() != heads:
            raise KernelError(f"a slope per query head: {heads} numbers, got {slopes.numel()}")
    g_ptr, g_splits, g_stride, g_row = c_void_p(0), 0, 0, 0
    if gate is not None:
        g_ptr, g_splits, g_stride, g_row, g_cols = _projection_view(gate)
        if g_cols != (heads if gate_per_head else heads * head_dim) or gate.shape[1] != n_tokens:
            raise KernelError("attention_tcgen05: the gate does not fit the heads")
    if not attention_tcgen05_supports(q.dtype, heads, kv_heads, head_dim):
        raise KernelError(f"the tcgen05 attention kernel does not take {q.dtype}, {heads}/{kv_heads} heads of size {head_dim}")
    if not (k_pool.dtype == v_pool.dtype == out.dtype == torch.bfloat16) or not q.is_contiguous():
        raise KernelError("queries, cache and output must all be contiguous bfloat16")
    fn = _fn("attention_tcgen05", "tt_attention_tcgen05", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                                                           c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p, c_void_p, c_float,
                                                           c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p])
    _check(fn(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(table), table.shape[1], k_pool.shape[0], _ptr(cu), _ptr(len_before), sequences,
              n_tokens, heads, kv_heads, head_dim, scale, _ptr(sinks), window, _ptr(out), _ptr(status), float(softcap or 0.0), _ptr(slopes),
              g_ptr, g_splits, g_stride, g_row, 1 if gate_per_head else 0, _stream()), "attention_tcgen05")


# --------------------------------------------------------------------------- recurrent
def _projection(proj: torch.Tensor) -> tuple:
    """(pointer, splits, split stride, columns) of float32 partial sums [splits, tokens, cols]."""
    _need(proj, torch.float32, "projection")
    if proj.dim() != 3:
        raise KernelError("a projection's partial sums are [splits, tokens, cols]")
    return _ptr(proj), proj.shape[0], proj.stride(0), proj.shape[2]


def _projection_view(proj: torch.Tensor) -> tuple:
    """(pointer, splits, split stride, row stride, columns) of float32 partial sums [splits, tokens, cols] that may be a
    range of the columns of a wider projection (``wide[:, :, a:b]``)."""
    if proj.dtype != torch.float32 or proj.dim() != 3 or proj.stride(2) != 1:
        raise KernelError("a projection's partial sums are float32 [splits, tokens, cols] with the columns side by side")
    return _ptr(proj), proj.shape[0], proj.stride(0), proj.stride(1), proj.shape[2]


def causal_conv(proj: torch.Tensor, col_off: int, channels: int, weight: torch.Tensor, bias: torch.Tensor | None, activation: bool,
                state: torch.Tensor, out: torch.Tensor, cu: torch.Tensor, slots: torch.Tensor, sequences: int, n_tokens: int,
                one_token_each: bool) -> None:
    """out[t, c] = f(bias[c] + sum_j weight[c, j] * x[t - (taps - 1) + j, c]) over each sequence's tokens, x being
    columns ``col_off .. col_off + channels`` of ``proj``; inputs before the step's first token come from ``state``
    [slots, taps - 1, channels] (float32, oldest first), which is moved on to the step's last inputs.  f is silu
    (``activation``) or the identity."""
    _need(weight, torch.float32, "convolution weight")
    _need(state, torch.float32, "convolution state")
    _need(out, torch.float32, "convolution output")
    taps = weight.shape[1]
    if weight.shape[0] != channels or tuple(state.shape[1:]) != (taps - 1, channels) or tuple(out.shape) != (n_tokens, channels):
        raise KernelError(f"convolution: weight {tuple(weight.shape)}, state {tuple(state.shape)}, out {tuple(out.shape)} do not fit {channels} channels")
    if bias is not None:
        _need(bias, torch.float32, "convolution bias")
    p, splits, stride, cols = _projection(proj)
    if col_off < 0 or col_off + channels > cols:
        raise KernelError("convolution: the channels lie outside the projection")
    fn = _fn("recurrent", "tt_causal_conv", [c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                             c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(p, splits, stride, cols, col_off, channels, _ptr(weight), _ptr(bias), taps, 1 if activation else 0, _ptr(state),
              state.stride(0) if state.numel() else 0, _ptr(out), _ptr(cu), _ptr(slots), sequences, n_tokens, 1 if one_token_each else 0,
              _stream()), "causal_conv", (0 if one_token_each else 1) + (1 if taps > 1 or one_token_each else 0))


SCAN_FORMS = {"auto": 0, "narrow": 1, "wide": 2}


def mamba2_scan(xbc: torch.Tensor, proj: torch.Tensor, dt_col: int, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
                state: torch.Tensor, y: torch.Tensor, cu: torch.Tensor, slots: torch.Tensor, sequences: int, heads: int,
                head_dim: int, state_size: int, groups: int, form: str = "auto") -> None:
    """The Mamba-2 recurrence over each sequence's tokens.  ``xbc`` float32 [tokens, inner + 2 * groups * state_size]
    holds x, B and C; column ``dt_col + h`` of ``proj`` the raw step size of head h; ``state`` float32
    [slots, heads, head_dim, state_size]; ``y`` float32 [tokens, inner] receives S^T C + D x.  ``form``: ``auto`` takes
    the form with one column per lane group unless that grid would fill the GPU more than twice over, then the one with
    four (``narrow`` / ``wide`` force one; both give the same bits, a column's arithmetic is the same)."""
    inner = heads * head_dim
    for t, name in ((xbc, "x/B/C"), (dt_bias, "dt_bias"), (a_log, "A_log"), (d_skip, "D"), (state, "recurrent state"), (y, "recurrence output")):
        _need(t, torch.float32, name)
    if xbc.shape[1] != inner + 2 * groups * state_size or tuple(state.shape[1:]) != (heads, head_dim, state_size) or y.shape[1] != inner:
        raise KernelError("mamba2_scan: shapes do not fit the sizes")
    p, splits, stride, cols = _projection(proj)
    fn = _fn("recurrent", "tt_mamba2_scan", [c_void_p, c_int, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(xbc), xbc.shape[1], p, splits, stride, cols, dt_col, _ptr(dt_bias), _ptr(a_log), _ptr(d_skip), _ptr(state), _ptr(y),
              _ptr(cu), _ptr(slots), sequences, heads, head_dim, state_size, groups, SCAN_FORMS[form], _stream()), "mamba2_scan")


def delta_scan(qkv: torch.Tensor, proj: torch.Tensor, b_col: int, a_col: int, dt_bias: torch.Tensor, a_log: torch.Tensor,
               state: torch.Tensor, out: torch.Tensor, cu: torch.Tensor, slots: torch.Tensor, sequences: int, heads: int, qk_heads: int,
               key_dim: int, value_dim: int, form: str = "auto") -> None:
    """The gated delta rule over each sequence's tokens.  ``qkv`` float32 [tokens, 2 * qk_heads * key_dim + heads *
    value_dim] holds q, k, v (q and k are made unit vectors here, q also times key_dim^-1/2); columns ``b_col + h`` and
    ``a_col + h`` of ``proj`` the raw write strength and decay input of head h; ``state`` float32
    [slots, heads, value_dim, key_dim]; ``out`` float32 [tokens, heads * value_dim] receives S^T q.  ``form``: as for
    :func:`mamba2_scan`."""
    for t, name in ((qkv, "q/k/v"), (dt_bias, "dt_bias"), (a_log, "A_log"), (state, "recurrent state"), (out, "recurrence output")):
        _need(t, torch.float32, name)
    if (qkv.shape[1] != 2 * qk_heads * key_dim + heads * value_dim or tuple(state.shape[1:]) != (heads, value_dim, key_dim)
            or out.shape[1] != heads * value_dim):
        raise KernelError("delta_scan: shapes do not fit the sizes")
    p, splits, stride, cols = _projection(proj)
    fn = _fn("recurrent", "tt_delta_scan", [c_void_p, c_int, c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                            c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(qkv), qkv.shape[1], p, splits, stride, cols, b_col, a_col, _ptr(dt_bias), _ptr(a_log), _ptr(state), _ptr(out),
              _ptr(cu), _ptr(slots), sequences, heads, qk_heads, key_dim, value_dim, SCAN_FORMS[form], _stream()), "delta_scan")


NORM_GATES = {"silu": 0, "sigmoid": 1}


def gated_group_norm(y: torch.Tensor, group: int, proj: torch.Tensor, gate_col: int, weight: torch.Tensor, eps: float, gate_first: bool,
                     out: torch.Tensor, gate: str = "silu") -> None:
    """Groups of ``group`` neighbouring columns of ``y`` (float32 [tokens, width]) divided by their root mean square,
    times ``weight`` (indexed by column modulo its length), with the gate silu(columns ``gate_col ..`` of ``proj``)
    multiplied in before the norm (``gate_first``) or after it; ``gate="sigmoid"`` takes the logistic function of the
    columns instead of silu."""
    if gate not in NORM_GATES:
        raise KernelError(f"the gate of a normed read-out is one of {sorted(NORM_GATES)}, not {gate!r}")
    _need(y, torch.float32, "norm input")
    _need(weight, torch.float32, "norm weight")
    tokens, width = y.shape
    if tuple(out.shape) != (tokens, width) or not out.is_contiguous() or width % group:
        raise KernelError("gated_group_norm: shapes do not fit")
    p, splits, stride, cols = _projection(proj)
    if gate_col + width > cols:
        raise KernelError("gated_group_norm: the gate lies outside the projection")
    fn = _fn("recurrent", "tt_gated_group_norm", [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p, c_int,
                                                  c_float, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(y), tokens, width, group, p, splits, stride, cols, gate_col, _ptr(weight), weight.numel(), eps, 1 if gate_first else 0,
              _ptr(out), dtype_code(out.dtype), NORM_GATES[gate], _stream()), "gated_group_norm")


def linear_attention_prepare(proj: torch.Tensor, heads: int, key_dim: int, value_dim: int, activation: bool, inv_freq: torch.Tensor | None,
                             rotary_dim: int, k_scale: float, vkq: torch.Tensor, cu: torch.Tensor, len_before: torch.Tensor,
                             sequences: int, n_tokens: int) -> None:
    """q, k and v of a linear attention from the partial sums of its input projection (columns ``[q | k | v | ...]``) as
    :func:`decay_scan` reads them, ``vkq`` float32 ``[tokens, heads * value_dim + 2 * heads * key_dim]``: silu on all three
    (``activation``), the first ``rotary_dim`` numbers of each head of q and k rotated by the position (halves paired), k times
    ``k_scale``."""
    _need(vkq, torch.float32, "v/k/q")
    if tuple(vkq.shape) != (n_tokens, heads * value_dim + 2 * heads * key_dim):
        raise KernelError("linear_attention_prepare: the output does not fit the sizes")
    if rotary_dim:
        _need(inv_freq, torch.float32, "inverse frequencies")
        if inv_freq.numel() < rotary_dim // 2:
            raise KernelError("linear_attention_prepare: too few inverse frequencies")
    p, splits, stride, cols = _projection(proj)
    fn = _fn("recurrent", "tt_linear_attention_prepare", [c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                                          c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(fn(p, splits, stride, cols, heads, key_dim, value_dim, 1 if activation else 0, _ptr(inv_freq) if rotary_dim else c_void_p(0),
              rotary_dim, k_scale, _ptr(vkq), _ptr(cu), _ptr(len_before), sequences, n_tokens, _stream()), "linear_attention_prepare")


def decay_scan(vkq: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, out: torch.Tensor, cu: torch.Tensor, slots: torch.Tensor,
               sequences: int, heads: int, key_dim: int, value_dim: int, form: str = "auto") -> None:
    """Linear attention with a fixed decay per head over each sequence's tokens: ``S = decay_h * S + k v^T``, ``o = S^T q``.
    ``vkq`` float32 ``[tokens, heads * value_dim + 2 * heads * key_dim]`` (v, k, q); ``decay`` float32 ``[heads]``; ``state``
    float32 ``[slots, heads, value_dim, key_dim]``; ``out`` float32 ``[tokens, heads * value_dim]``.  ``form``: as for
    :func:`mamba2_scan`, whose kernel this runs with a constant decay and step size one."""
    for t, name in ((vkq, "v/k/q"), (decay, "decay"), (state, "recurrent state"), (out, "recurrence output")):
        _need(t, torch.float32, name)
    if (vkq.shape[1] != heads * value_dim + 2 * heads * key_dim or tuple(state.shape[1:]) != (heads, value_dim, key_dim)
            or out.shape[1] != heads * value_dim or decay.numel() != heads):
        raise KernelError("decay_scan: shapes do not fit the sizes")
    fn = _fn("recurrent", "tt_decay_scan", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                            c_int, c_void_p])
    _check(fn(_ptr(vkq), vkq.shape[1], _ptr(decay), _ptr(state), _ptr(out), _ptr(cu), _ptr(slots), sequences, heads, value_dim, key_dim,
              SCAN_FORMS[form], _stream()), "decay_scan")


def weighted_pair(a: torch.Tensor, wa: float, b: torch.Tensor, wb: float, out: torch.Tensor) -> None:
    """out = wa * sum(a over its first axis) + wb * sum(b over its first axis), all float32."""
    for t, name in ((a, "first branch"), (b, "second branch"), (out, "sum")):
        _need(t, torch.float32, name)
    if a.shape[1:] != b.shape[1:] or out.numel() != a[0].numel():
        raise KernelError("weighted_pair: shapes differ")
    fn = _fn("recurrent", "tt_weighted_pair", [c_void_p, c_int, c_longlong, c_float, c_void_p, c_int, c_longlong, c_float, c_void_p, c_longlong, c_void_p])
    _check(fn(_ptr(a), a.shape[0], a.stride(0), wa, _ptr(b), b.shape[0], b.stride(0), wb, _ptr(out), out.numel(), _stream()), "weighted_pair")


# --------------------------------------------------------------------- latent attention
LATENT_MAX_RANK, LATENT_MAX_ROW, LATENT_MAX_DIM = 512, 1024, 256


def latent_prepare(down: torch.Tensor, q_rank: int, rank: int, rot: int, q_weight: torch.Tensor, kv_weight: torch.Tensor, eps: float,
                   inv_freq: torch.Tensor, rotary_dim: int, q_latent: torch.Tensor | None, pool: torch.Tensor | None, table: torch.Tensor,
                   cu: torch.Tensor, len_before: torch.Tensor, sequences: int, n_tokens: int, status: torch.Tensor,
                   interleaved: bool = False, rot_scale: float = 1.0) -> None:
    """From the partial sums of a down projection ``[q latent | kv latent | shared rotated key]``: both latents divided by
    their root mean square (``eps`` inside the root) times their weights; the query latent goes to ``q_latent`` ``[tokens,
    q_rank]``, and ``[kv latent | key part rotated by the position]`` to the token's row of ``pool`` ``[blocks, 1, 64, rank +
    rot]`` (nothing is written without a pool).  ``q_rank`` 0: no query latent (``q_weight`` and ``q_latent`` None).  ``down``
    may be a range of a wider projection's columns.  ``interleaved``: the rotation pairs neighbours instead of halves;
    ``rot_scale`` multiplies cosines and sines."""
    for t, name in ((kv_weight, "latent norm"), (inv_freq, "inverse frequencies")):
        _need(t, torch.float32, name)
    p, splits, stride, row_stride, cols = _projection_view(down)
    if q_rank:
        _need(q_weight, torch.float32, "query latent norm")
        if tuple(q_latent.shape) != (n_tokens, q_rank) or not q_latent.is_contiguous():
            raise KernelError("latent_prepare: the query latent does not fit the sizes")
    elif pool is None:
        return                                          # nothing to norm and nothing to append
    if cols != q_rank + rank + rot:
        raise KernelError("latent_prepare: shapes do not fit the sizes")
    if pool is not None and (tuple(pool.shape[1:]) != (1, BLOCK_TOKENS, rank + rot) or (q_rank and pool.dtype != q_latent.dtype)):
        raise KernelError("latent_prepare: the pool must be [blocks, 1, 64, rank + rot] in the activations' dtype")
    if (cols + 32) * 4 > 48 * 1024:
        raise KernelError(f"latent_prepare: {cols} projected numbers per token are more than the kernel stages")
    fn = _fn("latent_attention", "tt_latent_prepare", [c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                                                       c_void_p, c_int, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                                                       c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p])
    code = dtype_code(q_latent.dtype if q_rank else pool.dtype)
    _check(fn(p, splits, stride, row_stride, q_rank, rank, rot, _ptr(q_weight), _ptr(kv_weight), eps, _ptr(inv_freq), rotary_dim,
              1 if interleaved else 0, float(rot_scale), _ptr(q_latent), code,
              _ptr(pool), code, _ptr(table), table.shape[1], 0 if pool is None else pool.shape[0], _ptr(cu), _ptr(len_before), sequences,
              n_tokens, _ptr(status), _stream()), "latent_prepare")


def latent_attention(q: torch.Tensor, w_key: torch.Tensor, w_value: torch.Tensor, pool: torch.Tensor, table: torch.Tensor, cu: torch.Tensor,
                     len_before: torch.Tensor, sequences: int, n_tokens: int, heads: int, dim: int, rot: int, vdim: int, rank: int,
                     inv_freq: torch.Tensor, rotary_dim: int, scale: float, window: int, splits: int, out: torch.Tensor,
                     absorbed: torch.Tensor, part_acc: torch.Tensor, part_ml: torch.Tensor, status: torch.Tensor,
                     tensor_cores: bool = False, interleaved: bool = False, rot_scale: float = 1.0,
                     head_gate: torch.Tensor | None = None) -> None:
    """Causal softmax attention over a latent cache.  ``q``: float32 partial sums ``[slices, tokens, heads * (dim + rot)]`` of
    the queries (per head ``dim`` unrotated numbers, then ``rot`` of which the first ``rotary_dim`` are rotated here);
    ``w_key`` ``[heads * dim, rank]`` and ``w_value`` ``[heads * vdim, rank]`` expand a latent into a head's keys and values;
    ``pool`` ``[blocks, 1, 64, rank + rot]`` holds per token the latent and the rotated key part all heads share.  Score of
    query i and key j: ``(q_plain . w_key_h c_j + q_rot . k_rot_j) * scale`` for ``0 <= i - j < window`` (``window`` 0: every
    earlier key); ``out`` ``[tokens, heads * vdim]``.  Scratch memory, all float32: ``absorbed`` ``[tokens * heads * (rank +
    rot)]`` for the queries with ``w_key`` folded in; ``part_acc`` ``[tokens * heads * splits * rank]`` and ``part_ml``
    ``[tokens * heads * splits * 2]`` for the ``splits`` slices the keys are cut into.  ``tensor_cores``: a step of one token per
    sequence whose sizes :func:`latent_decode_tensor_cores` takes runs both products on the tensor cores, with the heads of a
    token as the rows; ``splits`` must then cover every key a token can see in slices of ``LATENT_DECODE_SLICE`` keys.
    ``q`` may be a range of a wider projection's columns.  ``interleaved`` / ``rot_scale``: as in :func:`latent_prepare`.
    ``head_gate``: float32 partial sums ``[slices, tokens, heads]`` (possibly such a range); every head's output is multiplied
    by the sigmoid of its number."""
    if tensor_cores and (n_tokens != sequences or not latent_decode_tensor_cores(out.dtype, rank, rot)):
        raise KernelError("latent_attention: the tensor-core form is for steps of one token per sequence and sizes it takes")
    _need(inv_freq, torch.float32, "inverse frequencies")
    if rank > LATENT_MAX_RANK or rank + rot > LATENT_MAX_ROW or dim > LATENT_MAX_DIM:
        raise KernelError(f"latent attention takes latents of up to {LATENT_MAX_RANK}, rows of up to {LATENT_MAX_ROW} and "
                          f"{LATENT_MAX_DIM} unrotated numbers per head; got {rank}, {rank + rot}, {dim}")
    p, q_splits, q_stride, q_row, q_cols = _projection_view(q)
    g_ptr, g_splits, g_stride, g_row = c_void_p(0), 0, 0, 0
    if head_gate is not None:
        g_ptr, g_splits, g_stride, g_row, g_cols = _projection_view(head_gate)
        if g_cols != heads or head_gate.shape[1] != n_tokens:
            raise KernelError("latent_attention: the gate has one number per head and token")
    if (q_cols != heads * (dim + rot) or tuple(w_key.shape) != (heads * dim, rank) or tuple(w_value.shape) != (heads * vdim, rank)
            or w_key.dtype != w_value.dtype or not w_key.is_contiguous() or not w_value.is_contiguous()
            or tuple(pool.shape[1:]) != (1, BLOCK_TOKENS, rank + rot) or pool.dtype != out.dtype
            or tuple(out.shape) != (n_tokens, heads * vdim) or not out.is_contiguous()):
        raise KernelError("latent_attention: shapes do not fit the sizes")
    for t, name in ((absorbed, "folded queries"), (part_acc, "slice sums"), (part_ml, "slice maxima")):
        _need(t, torch.float32, name)
    if (absorbed.numel() < n_tokens * heads * (rank + rot) or part_acc.numel() < n_tokens * heads * splits * rank
            or part_ml.numel() < n_tokens * heads * splits * 2):
        raise KernelError("latent_attention: scratch memory is too small")
    fn = _fn("latent_attention", "tt_latent_attention", [c_void_p, c_int, c_longlong, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                                         c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                         c_void_p, c_int, c_int, c_float, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                         c_void_p, c_int, c_void_p, c_int, c_longlong, c_int, c_void_p, c_void_p])
    _check(fn(p, q_splits, q_stride, q_row, _ptr(w_key), _ptr(w_value), dtype_code(w_key.dtype), _ptr(pool), dtype_code(out.dtype), _ptr(table),
              table.shape[1], pool.shape[0], _ptr(cu), _ptr(len_before), sequences, n_tokens, heads, dim, rot, vdim, rank, _ptr(inv_freq),
              rotary_dim, 1 if interleaved else 0, float(rot_scale), scale, window, splits, _ptr(out), _ptr(absorbed), _ptr(part_acc),
              _ptr(part_ml), 2 if tensor_cores else 0, g_ptr, g_splits, g_stride, g_row, _ptr(status), _stream()), "latent_attention", 3)


LATENT_DECODE_SLICE = 64        # keys of one slice of the tensor-core decode form (LT_KEYS in csrc/latent_attention.cu)


def latent_decode_tensor_cores(dtype: torch.dtype, rank: int, rot: int) -> bool:
    """Whether :func:`latent_attention` can decode on the tensor cores: a bfloat16 cache whose latent and rotated part are
    multiples of 16 numbers and whose staged slice fits the shared memory."""
    if dtype != torch.bfloat16:
        return False
    fn = _functions.get("tt_latent_decode_mma_takes")
    if fn is None:
        fn = getattr(build.load("latent_attention"), "tt_latent_decode_mma_takes")
        fn.argtypes, fn.restype = [c_int, c_int, c_int], c_int
        _functions["tt_latent_decode_mma_takes"] = fn
    return bool(fn(BF16, rank, rot))


def latent_expand(pool: torch.Tensor, table: torch.Tensor, cu: torch.Tensor, len_before: torch.Tensor, sequences: int, window: int,
                  bound_blocks: int, heads: int, dim: int, rot: int, rank: int, plan: torch.Tensor, table_tmp: torch.Tensor,
                  x: torch.Tensor, keys: torch.Tensor, status: torch.Tensor) -> None:
    """First half of expanding the latents a step of prompts can see into per-head keys and values laid out like cache blocks:
    ``table_tmp`` (int32 ``[sequences, table width]``) names, for every sequence, the temporary block that stands for each
    cache block the step reads (-1 elsewhere); ``x`` ``[bound_blocks * 64, rank]`` receives those blocks' latents (zero rows where
    there is no token) for the product with ``[w_key; w_value]``, and ``keys`` ``[bound_blocks, heads, 64, dim + rot]`` the
    shared rotated part behind every head's ``dim`` numbers.  ``plan``: int32 scratch ``[2 * sequences + 1]``.
    ``bound_blocks`` must be at least the blocks the step can see (the kernel flags a bad shape otherwise)."""
    _need(plan, torch.int32, "expansion plan")
    _need(table_tmp, torch.int32, "temporary table")
    if (plan.numel() < 2 * sequences + 1 or tuple(table_tmp.shape) != tuple(table.shape) or tuple(x.shape) != (bound_blocks * BLOCK_TOKENS, rank)
            or tuple(keys.shape) != (bound_blocks, heads, BLOCK_TOKENS, dim + rot) or not (pool.dtype == x.dtype == keys.dtype)
            or tuple(pool.shape[1:]) != (1, BLOCK_TOKENS, rank + rot) or not x.is_contiguous() or not keys.is_contiguous()):
        raise KernelError("latent_expand: shapes do not fit the sizes")
    fn = _fn("latent_attention", "tt_latent_expand_plan", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(cu), _ptr(len_before), sequences, window, table.shape[1], bound_blocks, _ptr(plan), _ptr(table_tmp), _ptr(status), _stream()),
           "latent_expand_plan")
    fn = _fn("latent_attention", "tt_latent_gather", [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                                      c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(pool), dtype_code(pool.dtype), _ptr(table), table.shape[1], pool.shape[0], _ptr(cu), _ptr(len_before), sequences, _ptr(plan),
              bound_blocks, heads, dim, rot, rank, _ptr(x), _ptr(keys), _stream()), "latent_gather")


def latent_scatter(y: torch.Tensor, heads: int, dim: int, rot: int, vdim: int, keys: torch.Tensor, values: torch.Tensor) -> None:
    """Second half: ``y``, the float32 partial sums ``[slices, bound_blocks * 64, heads * dim + heads * vdim]`` of the gathered
    latents times ``[w_key; w_value]``, into the first ``dim`` numbers of every head's keys and into ``values``
    ``[bound_blocks, heads, vdim, 64]`` (transposed inside a block, like the cache's)."""
    p, splits, stride, cols = _projection(y)
    blocks = keys.shape[0]
    if (cols != heads * (dim + vdim) or y.shape[1] != blocks * BLOCK_TOKENS or tuple(keys.shape) != (blocks, heads, BLOCK_TOKENS, dim + rot)
            or tuple(values.shape) != (blocks, heads, vdim, BLOCK_TOKENS) or keys.dtype != values.dtype
            or not keys.is_contiguous() or not values.is_contiguous()):
        raise KernelError("latent_scatter: shapes do not fit the sizes")
    fn = _fn("latent_attention", "tt_latent_scatter", [c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                                                       c_void_p])
    _check(fn(p, splits, stride, blocks, heads, dim, rot, vdim, _ptr(keys), _ptr(values), dtype_code(keys.dtype), _stream()), "latent_scatter")


def latent_queries(q: torch.Tensor, heads: int, dim: int, rot: int, inv_freq: torch.Tensor, rotary_dim: int, cu: torch.Tensor,
                   len_before: torch.Tensor, sequences: int, n_tokens: int, out: torch.Tensor, interleaved: bool = False,
                   rot_scale: float = 1.0) -> None:
    """The queries of the expanded form: the partial sums ``q`` ``[slices, tokens, heads * (dim + rot)]`` (possibly a range of a
    wider projection's columns) summed, every head's last ``rot`` numbers rotated by the position (the first ``rotary_dim`` of
    them, halves or neighbours paired, cosines and sines times ``rot_scale``), narrowed to ``out``."""
    _need(inv_freq, torch.float32, "inverse frequencies")
    p, splits, stride, q_row, cols = _projection_view(q)
    if cols != heads * (dim + rot) or tuple(out.shape) != (n_tokens, cols) or not out.is_contiguous():
        raise KernelError("latent_queries: shapes do not fit the sizes")
    fn = _fn("latent_attention", "tt_latent_queries", [c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_float,
                                                       c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p])
    _check(fn(p, splits, stride, q_row, heads, dim, rot, _ptr(inv_freq), rotary_dim, 1 if interleaved else 0, float(rot_scale), _ptr(cu),
              _ptr(len_before), sequences, n_tokens, _ptr(out), dtype_code(out.dtype), _stream()), "latent_queries")


# ------------------------------------------------------------------ stream, side input, gates
def add_narrow(residual: torch.Tensor, delta: torch.Tensor | None, out: torch.Tensor) -> None:
    """residual += sum of the float32 slices ``delta`` [slices, tokens, hidden] (None: nothing to add); ``out`` = the stream
    in the activation dtype, for a part that reads the stream itself."""
    _need(residual, torch.float32, "residual")
    if tuple(out.shape) != tuple(residual.shape) or not out.is_contiguous():
        raise KernelError("add_narrow: the output has the stream's shape")
    p, splits, stride = c_void_p(0), 0, 0
    if delta is not None:
        p, splits, stride, cols = _projection(delta)
        if tuple(delta.shape[1:]) != tuple(residual.shape):
            raise KernelError("add_narrow: the delta does not fit the stream")
    fn = _fn("elementwise", "tt_add_narrow", [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_longlong, c_void_p])
    _check(fn(_ptr(residual), p, splits, stride, _ptr(out), dtype_code(out.dtype), residual.numel(), _stream()), "add_narrow")


def token_side_gate(x: torch.Tensor, table: torch.Tensor, col_off: int, tokens: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    """out[t, j] = gelu_tanh(sum of the float32 slices x[s, t, j]) * table[tokens[t], col_off + j] for j < dim."""
    p, splits, stride, dim = _projection(x)
    _need(tokens, torch.int32, "tokens")
    n = tokens.numel()
    if table.dim() != 2 or not table.is_contiguous() or x.shape[1] != n or tuple(out.shape) != (n, dim) or not out.is_contiguous():
        raise KernelError("token_side_gate: shapes do not fit")
    if col_off < 0 or col_off + dim > table.shape[1]:
        raise KernelError("token_side_gate: the slice lies outside the table's rows")
    fn = _fn("elementwise", "tt_token_side_gate", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int,
                                                   c_void_p, c_int, c_void_p, c_void_p])
    _check(fn(p, splits, stride, _ptr(table), dtype_code(table.dtype), table.shape[0], table.shape[1], col_off, _ptr(tokens), n, dim,
              _ptr(out), dtype_code(out.dtype), _ptr(status), _stream()), "token_side_gate")


def sigmoid_gate(y: torch.Tensor, gate: torch.Tensor, head_width: int = 0) -> None:
    """In place: y[t, c] *= sigmoid(sum of the float32 slices gate[s, t, c]), or with ``head_width`` > 0 one gate number per
    head, gate[s, t, c // head_width].  ``gate`` may be a range of a wider projection's columns."""
    g_ptr, g_splits, g_stride, g_row, g_cols = _projection_view(gate)
    if y.dim() != 2 or not y.is_contiguous() or gate.shape[1] != y.shape[0]:
        raise KernelError("sigmoid_gate: shapes do not fit")
    if g_cols != (y.shape[1] // head_width if head_width > 0 else y.shape[1]):
        raise KernelError("sigmoid_gate: the gate does not fit the columns")
    fn = _fn("elementwise", "tt_sigmoid_gate", [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p])
    _check(fn(_ptr(y), dtype_code(y.dtype), y.shape[0], y.shape[1], g_ptr, g_splits, g_stride, g_row, int(head_width), _stream()), "sigmoid_gate")


# ------------------------------------------------------------------------------ routing
ROUTE_MAX_EXPERTS = 512


def _route_options(experts: int, score: str, correction: torch.Tensor | None, group_score: str, renormalize: bool, extra: int) -> tuple:
    if score not in ("softmax", "sigmoid") or group_score not in ("max", "top2"):
        raise KernelError("routing scores are 'softmax' or 'sigmoid', group scores 'max' or 'top2'")
    if correction is not None:
        _need(correction, torch.float32, "the choice correction")
        if correction.numel() != experts:
            raise KernelError(f"a correction per expert: {experts} numbers, got {correction.numel()}")
    if not 0 <= extra <= 32:
        raise KernelError("up to 32 always-on gates")
    return (1 if score == "sigmoid" else 0, _ptr(correction), 1 if group_score == "top2" else 0, 0 if renormalize else 1, int(extra))


def route_topk(logits: torch.Tensor, top: int, groups: int, keep: int, gates: torch.Tensor, chosen: torch.Tensor,
               weights: torch.Tensor, score: str = "softmax", correction: torch.Tensor | None = None, group_score: str = "max",
               renormalize: bool = True, extra: int = 0) -> None:
    """Routing of a mixture of experts from the router's logits (float32 partial sums ``[slices, tokens, experts]``): scores
    are the softmax over all experts; experts form ``groups`` equal groups of neighbours, a group's score is its largest
    expert score, and only experts of the ``keep`` best groups can be chosen; the ``top`` largest of those are chosen (ties:
    the lower index) and weighted by score / (sum of the chosen scores + 1e-20).  ``chosen`` int32 and ``weights`` float32
    ``[tokens, top]``; ``gates`` float32 ``[tokens, experts]`` holds the same densely, zero for experts not chosen.
    ``score`` "sigmoid": scores are the logits' sigmoids.  ``correction`` (float32, one per expert) is added to the scores for
    the choice only (groups and experts); weights stay the scores.  ``group_score`` "top2": a group's score is the sum of its
    two largest choice scores.  ``renormalize`` off: the weights are the chosen scores themselves.  ``extra``: so many more
    logits follow the experts'; ``gates`` then has ``experts + extra`` columns, the last ones the sigmoids of those logits."""
    p, splits, stride, experts = _projection(logits)
    experts -= extra
    options = _route_options(experts, score, correction, group_score, renormalize, extra)
    tokens = logits.shape[1]
    _need(gates, torch.float32, "gates")
    _need(weights, torch.float32, "routing weights")
    _need(chosen, torch.int32, "chosen experts")
    if (experts > ROUTE_MAX_EXPERTS or not 1 <= top <= min(32, experts) or not 1 <= groups <= 32 or experts % groups
            or not 1 <= keep <= groups):
        raise KernelError(f"route_topk takes up to {ROUTE_MAX_EXPERTS} experts in up to 32 equal groups and up to 32 choices; got "
                          f"{experts} experts, {groups} groups of which {keep} stay, top {top}")
    if tuple(gates.shape) != (tokens, experts + extra) or tuple(chosen.shape) != (tokens, top) or tuple(weights.shape) != (tokens, top):
        raise KernelError("route_topk: outputs do not fit the sizes")
    fn = _fn("routing", "tt_route_topk", [c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                          c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(p, splits, stride, tokens, experts, top, groups, keep, _ptr(gates), _ptr(chosen), _ptr(weights), *options, _stream()),
           "route_topk")


def route_rows(x: torch.Tensor, w: torch.Tensor, top: int, groups: int, keep: int, gates: torch.Tensor, chosen: torch.Tensor,
               weights: torch.Tensor, score: str = "softmax", correction: torch.Tensor | None = None, group_score: str = "max",
               renormalize: bool = True, extra: int = 0) -> None:
    """:func:`route_topk` with the router's product ``x @ w.T`` (float32 sums) in front, in one kernel: ``x`` ``[tokens,
    hidden]`` and ``w`` ``[experts + extra, hidden]``, each float32 or bfloat16."""
    tokens, hidden = x.shape
    experts = w.shape[0] - extra
    options = _route_options(experts, score, correction, group_score, renormalize, extra)
    _need(gates, torch.float32, "gates")
    _need(weights, torch.float32, "routing weights")
    _need(chosen, torch.int32, "chosen experts")
    if not x.is_contiguous() or not w.is_contiguous() or w.shape[1] != hidden:
        raise KernelError("route_rows: the rows and the router's matrix must be contiguous and of one width")
    if not route_rows_takes(hidden, experts + extra):
        raise KernelError(f"route_rows stages a row of up to {ROUTE_MAX_HIDDEN} numbers, got {hidden}")
    if (experts > ROUTE_MAX_EXPERTS or not 1 <= top <= min(32, experts) or not 1 <= groups <= 32 or experts % groups
            or not 1 <= keep <= groups):
        raise KernelError(f"route_rows takes up to {ROUTE_MAX_EXPERTS} experts in up to 32 equal groups and up to 32 choices; got "
                          f"{experts} experts, {groups} groups of which {keep} stay, top {top}")
    if tuple(gates.shape) != (tokens, experts + extra) or tuple(chosen.shape) != (tokens, top) or tuple(weights.shape) != (tokens, top):
        raise KernelError("route_rows: outputs do not fit the sizes")
    fn = _fn("routing", "tt_route_rows", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                          c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(x), dtype_code(x.dtype), _ptr(w), dtype_code(w.dtype), hidden, tokens, experts, top, groups, keep, _ptr(gates),
              _ptr(chosen), _ptr(weights), *options, _stream()), "route_rows")


ROUTE_MAX_HIDDEN = 11000


def route_rows_takes(hidden: int, experts: int) -> bool:
    """Whether a token's row and its logits fit the shared memory :func:`route_rows` stages them in."""
    return (hidden + experts + 32) * 4 <= 48 * 1024 and hidden <= ROUTE_MAX_HIDDEN


def scale_expert_columns(act: torch.Tensor, width: int, gates: torch.Tensor, experts: int | None = None, shared_width: int = 0) -> None:
    """act[t, e * width + j] *= gates[t, e] for the ``experts * width`` leading columns of ``act`` (in place; columns behind
    them stay as they are).  ``experts``: fewer than ``gates`` has columns; with ``shared_width`` the next so many columns of
    ``act`` are multiplied by ``gates[t, experts]`` (the gate of an expert that every token uses)."""
    _need(gates, torch.float32, "gates")
    tokens, columns = gates.shape
    experts = columns if experts is None else int(experts)
    if act.dim() != 2 or act.shape[0] != tokens or act.shape[1] < experts * width + shared_width or act.stride(1) != 1:
        raise KernelError("scale_expert_columns: the activations do not fit the gates")
    if experts > columns or (shared_width and experts >= columns):
        raise KernelError("scale_expert_columns: too few gates a token")
    fn = _fn("routing", "tt_scale_expert_columns", [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(act), dtype_code(act.dtype), tokens, act.stride(0), width, experts, _ptr(gates), columns, int(shared_width), _stream()),
           "scale_expert_columns")


def expert_activation(gate_up: torch.Tensor, act: torch.Tensor, experts: int, width: int, shared_width: int, limit: float,
                      shared_limit: float, alpha: float, gates: torch.Tensor, shared_gated: bool) -> None:
    """The clamped gated unit of a mixture's experts with the routing weights applied: ``gate_up`` float32 partial sums
    ``[slices, tokens, 2 * cols]`` (gate columns first), ``cols = experts * width + shared_width``.  With ``g' = min(g, limit)``
    and ``u' = clamp(u, -limit, limit)``: ``act[t, c] = g' sigmoid(alpha g') (u' + 1) * gates[t, c // width]`` for the routed
    experts' columns; the always-on expert's columns behind them use ``shared_limit`` and ``gates[t, experts]`` (``shared_gated``)
    or no weight.  A limit of 0 or less: no clamp."""
    p, splits, stride, cols2 = _projection(gate_up)
    _need(gates, torch.float32, "gates")
    tokens = gate_up.shape[1]
    cols = experts * width + shared_width
    if cols2 != 2 * cols or tuple(act.shape) != (tokens, cols) or not act.is_contiguous() or gates.shape[0] != tokens:
        raise KernelError("expert_activation: shapes do not fit the sizes")
    if gates.shape[1] < experts + (1 if shared_gated else 0):
        raise KernelError("expert_activation: too few gates a token")
    fn = _fn("routing", "tt_expert_activation", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                                 c_float, c_void_p, c_int, c_int, c_void_p])
    _check(fn(p, splits, stride, _ptr(act), dtype_code(act.dtype), tokens, experts, width, shared_width, float(limit or 0.0),
              float(shared_limit or 0.0), float(alpha), _ptr(gates), gates.shape[1], 1 if shared_gated else 0, _stream()), "expert_activation")


# -------------------------------------------------------------------------------- gemm
def gemm_simt(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor) -> None:
    """out[s] = x @ w[:, k-slice s].T in float32 FMA; ``out`` is float32
    [splits, m, n]; bias (float32 [n]) goes into slice 0."""
    _need(out, torch.float32, "gemm output")
    if x.stride(-1) != 1 or w.stride(-1) != 1:
        raise KernelError("gemm operands must be contiguous along k")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[1:] != (m, n):
        raise KernelError(f"gemm shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    fn = _fn("gemm_simt", "tt_gemm_simt", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_longlong,
                                           c_longlong, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(_ptr(x), dtype_code(x.dtype), x.stride(0), _ptr(w), dtype_code(w.dtype), w.stride(0), _ptr(bias), _ptr(out), out.stride(1),
              out.stride(0), m, n, k, out.shape[0], _stream()), "gemm_simt")


# ---------------------------------------------------------------------------- sampling
_argmax_scratch: dict[torch.device, tuple[torch.Tensor, torch.Tensor]] = {}


def argmax_rows(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[i] = argmax of logits[i], lowest id on ties.  Large vocabularies are reduced in
    two stages through a small scratch buffer kept per device."""
    _need(logits, torch.float32, "logits")
    _need(out, torch.int32, "token output")
    rows = logits.shape[0]
    scratch = _argmax_scratch.get(logits.device)
    if scratch is None or scratch[0].numel() < rows * 32:
        count = max(rows, 256) * 32
        scratch = (torch.empty(count, dtype=torch.float32, device=logits.device), torch.empty(count, dtype=torch.int32, device=logits.device))
        _argmax_scratch[logits.device] = scratch
    fn = _fn("sampling", "tt_argmax_rows", [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    two_stage = logits.shape[1] >= 8192
    _check(fn(_ptr(logits), logits.stride(0), rows, logits.shape[1], _ptr(out), _ptr(scratch[0]), _ptr(scratch[1]), _stream()),
           "argmax_rows", 2 if two_stage else 1)


def sample_rows(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int, request: torch.Tensor,
                step: torch.Tensor, out: torch.Tensor) -> None:
    _need(logits, torch.float32, "logits")
    _need(request, torch.int32, "request ids")
    _need(step, torch.int32, "step ids")
    _need(out, torch.int32, "token output")
    fn = _fn("sampling", "tt_sample_rows", [c_void_p, c_longlong, c_int, c_int, c_float, c_int, c_float, c_ulonglong, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(fn(_ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], temperature, top_k, top_p, seed & ((1 << 64) - 1),
              _ptr(request), _ptr(step), _ptr(out), _stream()), "sample_rows")


# ----------------------------------------------------------------- tensor-core kernels
_sm_counts: dict[int, int] = {}


def sm_count(device: torch.device | int | None = None) -> int:
    """Streaming multiprocessors of a CUDA device (the current one by default), asked of the device
    once: it sizes the k-slices of few-token products and the key slices of decode attention, which
    the launchers in C++ size from the same attribute."""
    index = torch.cuda.current_device() if device is None else (device if isinstance(device, int) else (device.index if device.index is not None else torch.cuda.current_device()))
    count = _sm_counts.get(index)
    if count is None:
        count = _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return count


SKINNY_TOKENS = 128         # up to this many tokens the weights go on the 128-row side of the tile


def gemm_tcgen05_usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    """TMA needs 16-byte aligned bases and row strides, i.e. k and both leading
    dimensions must be multiples of 8 bfloat16 numbers."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and x.stride(1) == 1 and w.stride(1) == 1)


PERSISTENT_TILES = 8        # from this many 128 x 256 output tiles on, prompts run the persistent kernel
PAIR_TOKENS = 2048          # from this many tokens on, CTA pairs run them, which do not slice k
PERSISTENT_SLICE_BLOCKS = 8  # a k-slice of the persistent kernel has at least this many 64-wide k-blocks


def gemm_tcgen05_splits(tokens: int, features: int, k: int, sms: int | None = None) -> int:
    """Into how many slices k is cut so that few output tiles still fill the GPU.  Few tokens:
    about two CTAs per SM, at least four 64-wide k-blocks per slice, at most 16 slices.
    Prompts (more than 128 tokens) with at least 8 tiles of 128 x 256 run the persistent kernel,
    one CTA per SM: as many slices as keep its work items within one round of the SMs (a
    512-token prompt has 32 tiles in the 1B shape's output projection), none of them empty.
    ``sms``: the device's multiprocessors (asked of the current device when not given)."""
    sms = sm_count() if sms is None else sms
    k_blocks = -(-k // 64)
    if tokens > SKINNY_TOKENS and -(-tokens // 128) * -(-features // 256) >= PERSISTENT_TILES:
        if tokens >= PAIR_TOKENS:
            return 1
        tiles = -(-tokens // 128) * -(-features // 256)
        if tiles * 8 <= sms:                  # tiles of 128 features where those of 256 fill at most an eighth of the SMs (the launcher does the same)
            tiles = -(-tokens // 128) * -(-features // 128)
        splits = max(1, min(sms // tiles, k_blocks // PERSISTENT_SLICE_BLOCKS, 16))
        while splits > 1 and (splits - 1) * -(-k_blocks // splits) >= k_blocks:
            splits -= 1
        return splits
    tiles = -(-features // 128) * (1 if tokens <= SKINNY_TOKENS else -(-tokens // 128))
    return max(1, min(2 * sms // tiles, k_blocks // 4, 16))


def gemm_tcgen05_accumulates(tokens: int, features: int, k: int, sms: int | None = None) -> bool:
    """Whether the product of these sizes can be added into its output by the kernel itself: prompts
    on the persistent or CTA-pair kernel whose k is not cut into slices, so that every output tile
    has one writer."""
    return (tokens > SKINNY_TOKENS and -(-tokens // 128) * -(-features // 256) >= PERSISTENT_TILES
            and gemm_tcgen05_splits(tokens, features, k, sms) == 1)


def gemm_tcgen05_accumulate_pays(tokens: int, features: int, k: int, sms: int | None = None) -> bool:
    """Whether adding into the output inside the kernel is also the faster way.  Where the output's rows are a multiple
    of 16 bytes the tiles are added by tiled copies from shared memory, which read nothing back, and the norm after the
    product then reads the stream alone: taken wherever it can be (measured on a B200 with the 1B shape's output and down
    projections, whole prefill: 2,048 tokens 3.98 -> 3.91 ms, 4,096 tokens 8.62 -> 8.51).  Other widths add from
    registers after reading the old values, which pays only where every CTA (or CTA pair) has at least two tiles, so
    that a tile's epilogue runs under the next tile's products."""
    sms = sm_count() if sms is None else sms
    if not gemm_tcgen05_accumulates(tokens, features, k, sms):
        return False
    if features % 4 == 0:
        return True
    if tokens >= PAIR_TOKENS:
        return -(-tokens // 256) * -(-features // 256) >= 2 * (sms // 2)
    return -(-tokens // 128) * -(-features // 256) >= 2 * sms


_shares_words: dict[int, int] = {}


def gemm_tcgen05_shares_words() -> int:
    """int32 words of scratch memory with which the CTA pairs of a prompt's plain product may deal the tiles' k-blocks out
    evenly among themselves (``shares`` of :func:`gemm_tcgen05`): a share of a tile per epilogue warp, and a flag word
    each at the end, which must be zero before a call and is zero again after it."""
    device = torch.cuda.current_device()
    words = _shares_words.get(device)
    if words is None:
        lib = build.load("gemm_tcgen05")
        lib.tt_gemm_tcgen05_shares_bytes.argtypes = []
        lib.tt_gemm_tcgen05_shares_bytes.restype = c_longlong
        words = _shares_words[device] = int(lib.tt_gemm_tcgen05_shares_bytes()) // 4
    return words


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor, status: torch.Tensor,
                 operands_checked: bool = False, accumulate: bool = False, shares: torch.Tensor | None = None) -> None:
    """out[s] = x @ w[:, k-slice s].T on the tensor cores; bfloat16 operands, float32
    ``out`` [splits, tokens, features]; bias (float32) goes into slice 0.  ``operands_checked``: the
    caller has already called :func:`gemm_tcgen05_usable` on these operands.  ``accumulate``: the
    product is added to ``out`` [1, tokens, features] (only where :func:`gemm_tcgen05_accumulates`).
    ``shares``: zeroed int32 scratch memory of :func:`gemm_tcgen05_shares_words` words; with it, prompts on
    CTA pairs whose tiles would leave pairs idle share the tiles' k among the pairs."""
    _need(out, torch.float32, "gemm output")
    tokens, k = x.shape
    features = w.shape[0]
    if accumulate and (out.shape[0] != 1 or not gemm_tcgen05_accumulates(tokens, features, k)):
        raise KernelError(f"tcgen05 gemm cannot add a product of {tokens} x {features} x {k} into its output")
    if not (operands_checked or gemm_tcgen05_usable(x, w)) or w.shape[1] != k or tuple(out.shape[1:]) != (tokens, features):
        raise KernelError(f"tcgen05 gemm cannot take x {tuple(x.shape)} / w {tuple(w.shape)} / out {tuple(out.shape)} (k and strides must be multiples of 8)")
    if out.shape[0] > -(-k // 64):
        raise KernelError(f"{out.shape[0]} k-slices for k = {k}: a slice needs at least one block of 64")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    if shares is not None and (shares.dtype != torch.int32 or not shares.is_contiguous()):
        raise KernelError("the shares of a tcgen05 gemm must be contiguous int32")
    fn = _fn("gemm_tcgen05", "tt_gemm_tcgen05", [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_longlong,
                                                 c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_longlong])
    _check(fn(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out), out.stride(1), out.stride(0), tokens, features, k,
              out.shape[0], 2 if accumulate else 0, _ptr(status), _stream(), _ptr(shares), 0 if shares is None else shares.numel() * 4),
           "gemm_tcgen05")


def gemm_tcgen05_qkv_rope_takes(x: torch.Tensor, w: torch.Tensor, head_dim: int, rotary_dim: int) -> bool:
    """Whether the qkv product of these operands can rotate, narrow and append to the cache in its own epilogue:
    a prompt on the persistent or CTA-pair kernel without k-slices, head size 64 or 128 rotated whole."""
    if rotary_dim != head_dim or head_dim not in (64, 128) or not gemm_tcgen05_usable(x, w):
        return False
    lib = build.load("gemm_tcgen05")
    lib.tt_gemm_tcgen05_qkv_rope_takes.argtypes = [c_int, c_int, c_int, c_int]
    lib.tt_gemm_tcgen05_qkv_rope_takes.restype = c_int
    return bool(lib.tt_gemm_tcgen05_qkv_rope_takes(x.shape[0], w.shape[0], x.shape[1], head_dim))


def gemm_tcgen05_qkv_rope(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, q_out: torch.Tensor, k_pool: torch.Tensor,
                          v_pool: torch.Tensor, cos_sin: torch.Tensor, where: torch.Tensor, table: torch.Tensor, heads: int,
                          kv_heads: int, head_dim: int, attention_scaling: float, status: torch.Tensor) -> None:
    """The qkv projection of a prompt with the rotation, the narrowing to bfloat16 and the cache append done by the
    product's epilogue: q (rotated) to ``q_out`` [tokens, heads * head_dim], k (rotated) and v into the block pools at
    each token's position.  ``cos_sin`` and ``where`` are the step's :func:`rope_table`.  Only where
    :func:`gemm_tcgen05_qkv_rope_takes`."""
    tokens, k = x.shape
    q_cols, kv_cols = heads * head_dim, kv_heads * head_dim
    if w.shape != (q_cols + 2 * kv_cols, k) or tuple(q_out.shape) != (tokens, q_cols):
        raise KernelError(f"qkv product: w {tuple(w.shape)} / q_out {tuple(q_out.shape)} do not fit {heads}/{kv_heads} heads of {head_dim}")
    for t, name in ((q_out, "q_out"), (k_pool, "key pool"), (v_pool, "value pool")):
        _need(t, torch.bfloat16, name)
    if bias is not None:
        _need(bias, torch.float32, "bias")
    _need(cos_sin, torch.float32, "cos/sin table")
    _need(where, torch.int32, "token positions")
    if tuple(cos_sin.shape) != (tokens, head_dim // 2, 2) or tuple(where.shape) != (tokens, 2):
        raise KernelError("qkv product: the rope table does not fit the step")
    fn = _fn("gemm_tcgen05", "tt_gemm_tcgen05_qkv_rope", [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                                          c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                                          c_void_p, c_void_p])
    code = fn(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(bias), tokens, k, _ptr(q_out), _ptr(k_pool), _ptr(v_pool), _ptr(cos_sin),
              _ptr(where), _ptr(table), table.shape[1], k_pool.shape[0], heads, kv_heads, head_dim, attention_scaling, _ptr(status), _stream())
    if code < 0:
        raise KernelError("qkv product with rotation: " + ("a tensor map could not be made" if code == -1 else "the shape is not taken"))
    _check(code, "gemm_tcgen05_qkv_rope")


def gemm_tcgen05_failure_drill(wait_limit_ns: int, undelivered_bytes: int) -> None:
    """For tests of the failure path, never for serving.  ``wait_limit_ns``: the limit of every
    bounded wait in the tensor-core product kernels (0 restores the default of two seconds).
    ``undelivered_bytes``: from now on the first stage of the few-token and small-prompt kernel
    expects that many bytes more than its copies bring (0 restores normal operation), so its
    barrier never completes; the kernel must then raise ``STATUS_WAIT_EXPIRED``, free what it
    holds and return."""
    lib = build.load("gemm_tcgen05")
    lib.tt_gemm_tcgen05_set_wait_limit_ns.argtypes = [c_ulonglong]
    lib.tt_gemm_tcgen05_set_wait_limit_ns.restype = c_int
    lib.tt_gemm_tcgen05_expect_undelivered_bytes.argtypes = [c_int]
    lib.tt_gemm_tcgen05_expect_undelivered_bytes.restype = None
    code = lib.tt_gemm_tcgen05_set_wait_limit_ns(int(wait_limit_ns))
    if code != 0:
        raise KernelError(f"setting the wait limit failed: CUDA error {code}")
    lib.tt_gemm_tcgen05_expect_undelivered_bytes(int(undelivered_bytes))


def gemm_tcgen05_swiglu(x: torch.Tensor, w: torch.Tensor, act: torch.Tensor, status: torch.Tensor, activation: str = "silu") -> None:
    """act = f(x @ gate.T) * (x @ up.T) in bfloat16, where ``w`` [2 * inter, k] holds
    the gate rows followed by the up rows and f is silu, relu or gelu_tanh; the activation never exists in float32 in
    global memory."""
    _need(act, torch.bfloat16, "activation output")
    if activation not in GATE_ACTIVATIONS:
        raise KernelError(f"gate activation {activation!r} is not one of {sorted(GATE_ACTIVATIONS)}")
    tokens, k = x.shape
    inter = w.shape[0] // 2
    if not gemm_tcgen05_usable(x, w) or w.shape[1] != k or tuple(act.shape) != (tokens, inter):
        raise KernelError(f"tcgen05 swiglu gemm cannot take x {tuple(x.shape)} / w {tuple(w.shape)} / act {tuple(act.shape)}")
    fn = _fn("gemm_tcgen05", "tt_gemm_tcgen05", [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_longlong,
                                                 c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_longlong])
    _check(fn(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(None), _ptr(act), act.stride(0), 0, tokens, inter, k, 1,
              1 + 16 * GATE_ACTIVATIONS[activation], _ptr(status), _stream(), _ptr(None), 0), "gemm_tcgen05_swiglu")


def gemm_tcgen05_clamped(x: torch.Tensor, w: torch.Tensor, act: torch.Tensor, status: torch.Tensor, limit: float, shared_limit: float,
                         split: int, alpha: float) -> None:
    """:func:`gemm_tcgen05_swiglu` with the clamped unit as its epilogue: with ``g' = min(g, limit)`` and ``u' = clamp(u, -limit,
    limit)``, ``act[t, f] = g' sigmoid(alpha g') (u' + 1)``; output features below ``split`` use ``limit``, the others
    ``shared_limit`` (0 or less: no clamp)."""
    _need(act, torch.bfloat16, "activation output")
    tokens, k = x.shape
    inter = w.shape[0] // 2
    if not gemm_tcgen05_usable(x, w) or w.shape[1] != k or tuple(act.shape) != (tokens, inter):
        raise KernelError(f"tcgen05 gated gemm cannot take x {tuple(x.shape)} / w {tuple(w.shape)} / act {tuple(act.shape)}")
    fn = _fn("gemm_tcgen05", "tt_gemm_tcgen05_clamped", [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int,
                                                         c_float, c_float, c_int, c_float, c_void_p, c_void_p])
    _check(fn(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(act), act.stride(0), tokens, inter, k, float(limit or 0.0),
              float(shared_limit or 0.0), int(split), float(alpha), _ptr(status), _stream()), "gemm_tcgen05_clamped")
