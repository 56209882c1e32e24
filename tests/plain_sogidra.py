"""Plain, slow implementation of the Sogidra decoder, used only as the test oracle.

Sogidra is a decoder with learned position vectors added to the token embedding and no rotation anywhere.  Every
sublayer stands between two RMS norms whose weights are stored around zero (``1 + w`` multiplies): the stream gets
``norm_after(sublayer(norm_before(x)))`` added.  After each layer the stream that goes on is a learned weighted sum of
the embedding output and of every layer's result so far.  A layer's mixer is one of two attentions: a *differential*
attention (two softmax maps per head over the same values, the second subtracted with a learned weight, the difference
normed per head; queries grow with the logarithm of the position; a layer may read an earlier layer's keys and values
instead of projecting its own), or a sliding-window attention whose values are its unnormed keys, with unit-norm
queries and keys, scores squashed by a tanh, and, beyond the window, one mean key and mean value per whole block of
tokens that has left the window.  The feed-forward is ``down(act(up x))`` with a two-parameter activation that is
quadratic for positive inputs and a scaled ``exp(z) - 1 - z`` for the others.  The output matrix is the embedding table.

Everything here works on one whole sequence at a time with explicit loops over positions where that is clearest, no
cache and no batching.  It shares no code with the package under test: own config reading, own safetensors reader, one
function per mechanism.  Arithmetic is float64.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

# What stands in for the narrowing of activations: None (exact), or a function applied wherever an engine that multiplies
# bfloat16 matrices narrows its operand (the input of every projection, cached keys and values, the heads' outputs).
_narrow = None


def nar(x):
    return x if _narrow is None else _narrow(x)


_NP = {"F32": np.float32, "F64": np.float64, "F16": np.float16, "I32": np.int32, "I64": np.int64}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """name -> float64 (or int64) tensor; bfloat16 is widened exactly."""
    data = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", data[:8])
    header = json.loads(data[8:8 + n].decode("utf-8"))
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = data[8 + n + lo:8 + n + hi]
        shape = tuple(meta["shape"])
        if meta["dtype"] == "BF16":
            words = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            array = words.view(np.float32).astype(np.float64)
        else:
            array = np.frombuffer(raw, dtype=np.dtype(_NP[meta["dtype"]]).newbyteorder("<"))
            array = array.astype(np.int64 if meta["dtype"].startswith("I") else np.float64)
        out[name] = torch.from_numpy(array.reshape(shape).copy())
    return out


def read_model(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


# ------------------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def zero_centred_norm(x, w, eps):
    """RMS norm whose stored weight is the distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def softplus(x):
    return math.log1p(math.exp(x))


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z/2.  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    up = softplus(p) * z * z + 0.5 * z
    down = (0.5 + softplus(q)) * (torch.exp(torch.clamp(z, max=0.0)) - 1.0 - z) + 0.5 * z
    return torch.where(z > 0, up, down)


def feed_forward(x, w, pre: str):
    act = w[pre + "act"]
    return nar(xielu(nar(x) @ w[pre + "up"].T, float(act[0]), float(act[1]))) @ w[pre + "down"].T


def embed(tokens, w):
    """Token row plus the learned vector of the position."""
    ids = torch.tensor(tokens, dtype=torch.long)
    return w["embed"][ids] + w["pos"][: len(tokens)]


def softmax_row(scores):
    e = torch.exp(scores - scores.max())
    return e / e.sum()


# ------------------------------------------------------------------------- differential attention
def query_temperature(position: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log((position + 1) // every + 1)


def differential_lambda(w, pre: str, diff: float) -> float:
    return math.exp(float((w[pre + "lq1"] * w[pre + "lk1"]).sum())) - math.exp(float((w[pre + "lq2"] * w[pre + "lk2"]).sum())) + diff


def differential_keys_values(x, m, w, pre: str):
    """Keys [T, G, 2, dim] and values [T, G, vdim] of a layer that projects its own."""
    T = x.shape[0]
    G, dim, vdim = m["kv_heads"], m["dim"], m["vdim"]
    k = nar(x) @ w[pre + "k"].T + w[pre + "k.b"]
    v = nar(x) @ w[pre + "v"].T + w[pre + "v.b"]
    return nar(k.view(T, G, 2, dim)), nar(v.view(T, G, vdim))


def differential_attention(x, m, w, pre: str, eps: float, keys, values):
    """``keys`` / ``values``: this layer's own, or those of the layer it reads."""
    T = x.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (nar(x) @ w[pre + "q"].T + w[pre + "q.b"]).view(T, H, 2, dim)
    lam = differential_lambda(w, pre, m["diff"])
    out = torch.zeros(T, H, vdim, dtype=x.dtype)
    for i in range(T):
        temp = query_temperature(i, m["q_temp"]["coef"], m["q_temp"]["every"]) if m.get("q_temp") else 1.0
        for h in range(H):
            g = h // (H // G)
            maps = []
            for which in range(2):
                scores = (keys[: i + 1, g, which] @ nar(q[i, h, which] * temp)) * m["scale"]
                maps.append(softmax_row(scores) @ values[: i + 1, g])
            o = maps[0] - lam * maps[1]
            out[i, h] = unit_rms(o, eps) * (1.0 - m["diff"])
    return nar(out.reshape(T, H * vdim)) @ w[pre + "o"].T


# ------------------------------------------------------------------------- window attention with pooled blocks
def visible_blocks(position: int, size: int, pool: int) -> int:
    """How many whole blocks of ``pool`` tokens lie before the window of ``position``: block b ends at
    b * pool + pool - 1, which must be at most position - size."""
    return max(0, (position - size + 1) // pool)


def pooled_window_attention(x, m, w, pre: str, eps: float):
    T = x.shape[0]
    H, G, dim = m["heads"], m["kv_heads"], m["dim"]
    size, pool = m["mask"]["size"], m["mask"]["pool"]
    cap = m.get("softcap")
    q = nar(unit_rms((nar(x) @ w[pre + "q"].T).view(T, H, dim), eps))
    raw = (nar(x) @ w[pre + "k"].T).view(T, G, dim)
    keys, values = nar(unit_rms(raw, eps)), nar(raw)
    blocks = T // pool
    key_means = nar(keys[: blocks * pool].view(blocks, pool, G, dim).mean(1))
    value_means = nar(values[: blocks * pool].view(blocks, pool, G, dim).mean(1))
    out = torch.zeros(T, H, dim, dtype=x.dtype)
    for i in range(T):
        first = max(0, i - size + 1)
        nb = visible_blocks(i, size, pool)
        for h in range(H):
            g = h // (H // G)
            ks = torch.cat([key_means[:nb, g], keys[first: i + 1, g]])
            vs = torch.cat([value_means[:nb, g], values[first: i + 1, g]])
            scores = (ks @ q[i, h]) * m["scale"]
            if cap:
                scores = cap * torch.tanh(scores / cap)
            out[i, h] = softmax_row(scores) @ vs
    return nar(out.reshape(T, H * dim)) @ w[pre + "o"].T


# ------------------------------------------------------------------------- the model
def forward(cfg, w, tokens, narrow=None, layers_out: list | None = None):
    """Logits [T, vocab] for one whole sequence; ``layers_out`` collects the stream after every layer."""
    global _narrow
    _narrow = narrow
    try:
        eps = cfg["norm"]["eps"]
        x = embed(tokens, w)
        results = [x]                                   # the embedding output, then every layer's result
        kept: dict[int, tuple] = {}                     # layer -> (keys, values) of a differential layer that projects
        for index, layer in enumerate(cfg["layers"]):
            pre = f"l{index}."
            m = layer["mixer"]
            h = zero_centred_norm(x, w[pre + "norm1"], eps)
            if layer["type"] == "attention":
                source = m.get("kv_from")
                if source is None:
                    kept[index] = differential_keys_values(h, m, w, pre + "mix.")
                    source = index
                mixed = differential_attention(h, m, w, pre + "mix.", eps, *kept[source])
            elif layer["type"] == "attention_2":
                mixed = pooled_window_attention(h, m, w, pre + "mix.", eps)
            else:
                raise ValueError(f"unknown layer type {layer['type']!r}")
            x = x + zero_centred_norm(mixed, w[pre + "norm1b"], eps)
            if layer.get("mlp") is not None:
                fed = feed_forward(zero_centred_norm(x, w[pre + "norm2"], eps), w, pre + "mlp.")
                x = x + zero_centred_norm(fed, w[pre + "norm2b"], eps)
            results.append(x)
            x = sum(float(w[pre + "dwa"][j]) * results[j] for j in range(index + 2))
            if layers_out is not None:
                layers_out.append(x)
        final = zero_centred_norm(x, w["final.norm"], eps)
        return nar(final) @ w["embed"].T
    finally:
        _narrow = None
