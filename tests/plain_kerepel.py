"""Plain, slow implementation of the Kerepel decoder, used only as the test oracle.

Kerepel is a pre-norm decoder, ``x += mixer(norm1(x)); x += ff(norm2(x))`` with RMS norms, whose layers end with a
*per-layer token input*: a slice of a second embedding of the token, gated by a small projection of the stream,
projected back, RMS-normed and added.  The embedding adds a hashed row for the (previous token, token) pair.  The mixer is
one of two, in an order config.json lists.  *Attention*: grouped heads whose q, k and v pass a short causal convolution
over time right after their projections, q and k an RMS norm per head, scores that are scaled, capped by a tanh and
lowered by ``slope_h * distance``, a sliding window, a sigmoid gate on the concatenated heads; a layer may read an earlier
layer's keys and values instead of projecting its own.  *Latent attention*: keys and values are expansions of one cached
latent per token plus one rotated key part shared by all heads (interleaved pairs, YaRN frequencies), full causal, one
sigmoid gate per head.  The feed-forward is ``down(gelu(up h))`` or a mixture of experts: sigmoid scores, a correction
added for the choice only, groups scored by their two best, weights not renormalised, clamped gated experts and a
gated shared expert.  The head is the embedding table times a constant.

Everything here works on one whole sequence at a time with no cache and no batching.  It shares no code with the
package under test: own config reading, own safetensors reader, one function per mechanism.  Arithmetic is float64 except
for the rotation's angles, which are float32 products of float32 factors like an engine's.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

# What stands in for the narrowing of activations: None (exact), or a function applied wherever an engine that
# multiplies bfloat16 matrices narrows its operand.  ``forward(..., narrow=f)`` sets it.
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
def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) (* w) over the last axis."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def short_convolution(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the sequence's start."""
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + u.shape[0]] * w[:, j]
    return y


def yarn_frequencies(rot):
    """Float32 frequencies of the pairs and the factor on cosines and sines."""
    dims, base = rot["dims"], float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    s = rot.get("scaling")
    if not s:
        return f.to(torch.float32), 1.0

    def turn(t):
        return dims * math.log(s["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn(s["fast"])), 0)
    hi = min(math.ceil(turn(s["slow"])), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    f = f / s["factor"] * ramp + f * (1.0 - ramp)
    return f.to(torch.float32), 0.1 * math.log(s["factor"]) + 1.0


def rotate_pairs(x, positions, rot):
    """Rotate the first ``dims`` numbers of the last axis of x [T, ..., n] in neighbouring pairs: (u, v) = (x[2i], x[2i+1])
    at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * f_i (a float32 product)."""
    dims = rot["dims"]
    f, factor = yarn_frequencies(rot)
    angle = (positions.to(torch.float32)[:, None] * f[None, :]).to(torch.float64)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = (torch.cos(angle) * factor).reshape(shape), (torch.sin(angle) * factor).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([u * cos - v * sin, v * cos + u * sin], dim=-1).reshape(*x.shape[:-1], dims)
    return torch.cat([turned, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------- embedding
def embed(tokens, table, bigram, spec):
    """Row ``token`` of the table plus the pair's hashed row of ``bigram``; a sequence's first token takes the last row."""
    x = table[tokens].clone()
    if spec is None:
        return x
    buckets, a, b = spec["buckets"], spec["mul_prev"], spec["mul_cur"]
    for t in range(len(tokens)):
        row = buckets if t == 0 else (int(tokens[t - 1]) * a + int(tokens[t]) * b) % buckets
        x[t] += bigram[row]
    return x


def token_side(x, tokens, w, p, index, dim, eps):
    """What the layer's own slice of the side table adds: rms(proj(gelu_tanh(gate x) * e)) * weight."""
    e = w["side.embed"][tokens][:, index * dim:(index + 1) * dim]
    g = gelu_tanh(nar(x) @ w[p + "gate"].T) * e
    y = nar(g) @ w[p + "proj"].T
    return rms_norm(y, w[p + "norm"], eps)


# ------------------------------------------------------------------------------- mixers
def attention_keys_values(h, w, p, m, eps):
    """Keys [T, G, D] after convolution and norm, values [T, G, V] after convolution."""
    T = h.shape[0]
    G, D, V = m["kv_heads"], m["dim"], m["vdim"]
    k, v = h @ w[p + "k"].T, h @ w[p + "v"].T
    if m.get("conv"):
        k, v = short_convolution(k, w[p + "k.conv"]), short_convolution(v, w[p + "v.conv"])
    k = rms_norm(k.reshape(T, G, D), w[p + "k.norm"], eps)
    return nar(k), nar(v.reshape(T, G, V))


def attention(h, w, p, m, eps, keys_values):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    h = nar(h)
    q = h @ w[p + "q"].T
    if m.get("conv"):
        q = short_convolution(q, w[p + "q.conv"])
    q = nar(rms_norm(q.reshape(T, H, D), w[p + "q.norm"], eps))
    k, v = keys_values
    cap = m.get("softcap")
    window = (m.get("mask") or {}).get("size")
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        slope = 2.0 ** (-8.0 * (head + 1) / H)
        for t in range(T):
            lo = 0 if not window else max(0, t - window + 1)
            s = (k[lo:t + 1, g] @ q[t, head]) * m["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            s = s - slope * (t - torch.arange(lo, t + 1, dtype=h.dtype))
            out[t, head] = torch.softmax(s, dim=0) @ v[lo:t + 1, g]
    out = out.reshape(T, H * V) * sigmoid(h @ w[p + "g"].T)
    return nar(out) @ w[p + "o"].T


def latent_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, D, R, V, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    h = nar(h)
    q = (h @ w[p + "q"].T).reshape(T, H, D + R)
    down = h @ w[p + "dkv"].T
    c = nar(rms_norm(down[:, :rank], w[p + "dkv.norm"], eps))
    q_plain, q_rot, k_rot = q[..., :D], q[..., D:], down[:, rank:]
    if m.get("rot"):
        q_rot, k_rot = rotate_pairs(q_rot, pos, m["rot"]), rotate_pairs(k_rot, pos, m["rot"])
    k_rot = nar(k_rot)
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, D)
    v = (c @ w[p + "uv"].T).reshape(T, H, V)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        s = (torch.einsum("hd,jhd->hj", q_plain[t], k_plain[:t + 1]) + q_rot[t] @ k_rot[:t + 1].T) * m["scale"]
        out[t] = torch.einsum("hj,jhv->hv", torch.softmax(s, dim=-1), v[:t + 1])
    out = out * sigmoid(h @ w[p + "g"].T)[:, :, None]
    return nar(out.reshape(T, H * V)) @ w[p + "o"].T


# ------------------------------------------------------------------------- feed-forward
def dense(h, w, p):
    return nar(gelu_erf(nar(h) @ w[p + "up"].T)) @ w[p + "down"].T


def clamped_expert(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, -limit, limit)
    return nar(g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(scores, correction, top, groups, keep):
    """One token's experts: the choice runs on score + correction among the experts of the ``keep`` groups whose two
    largest choice scores sum highest; the weights are the plain scores of the chosen."""
    E = scores.numel()
    size = E // groups
    choice = scores + correction
    best_two = torch.topk(choice.reshape(groups, size), min(2, size), dim=1).values.sum(dim=1)
    kept = sorted(range(groups), key=lambda g: (-float(best_two[g]), g))[:keep]
    allowed = [e for e in range(E) if e // size in kept]
    chosen = sorted(allowed, key=lambda e: (-float(choice[e]), e))[:top]
    return chosen, [scores[e] for e in chosen]


def mixture(h, w, p, mlp):
    r = mlp["router"]
    h = nar(h)
    groups = r.get("groups") or {"count": 1, "keep": 1}
    scores = sigmoid(h @ w[p + "router"].T)
    correction = w[p + "correction"] if p + "correction" in w else torch.zeros_like(scores[0])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        chosen, weights = route(scores[t], correction, r["top"], groups["count"], groups["keep"])
        for e, g in zip(chosen, weights):
            out[t] += g * clamped_expert(h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + sigmoid(h @ w[p + "shared.sg"].T) * clamped_expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


# -------------------------------------------------------------------------------- model
def forward(config, w, tokens, dtype=torch.float64, layers_out=None, narrow=None):
    """Logits [tokens, vocab] of one whole sequence.  ``layers_out``: a list that receives the stream after each layer."""
    global _narrow
    _narrow = narrow
    try:
        return _forward(config, w, tokens, dtype, layers_out)
    finally:
        _narrow = None


def _forward(config, w, tokens, dtype, layers_out):
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = config["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.int64)
    x = embed(tokens, w["embed"], w.get("bigram"), (config.get("embedding") or {}).get("bigram"))
    side = config.get("token_side")
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            source = m.get("kv_from")
            if source is None:
                kept[i] = attention_keys_values(nar(h), w, p + "mix.", m, eps)
            x = x + attention(h, w, p + "mix.", m, eps, kept[i if source is None else source])
        else:
            x = x + latent_attention(h, w, p + "mix.", m, eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            x = x + (dense(h, w, p + "mlp.") if mlp["kind"] == "dense" else mixture(h, w, p + "mlp.", mlp))
        if side:
            x = x + token_side(x, tokens, w, p + "side.", i, side["dim"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return (nar(rms_norm(x, w["final.norm"], eps)) @ w["embed"].T) * config.get("logit_scale", 1.0)
