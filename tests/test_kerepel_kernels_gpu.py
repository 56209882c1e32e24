"""The kernels behind the Kerepel parts, each alone against a plain float64 restatement written here, at other sizes
than the engine tests': attention with capped scores, distance slopes, a window and an output gate through a scrambled
cache, with one key made to dominate far away, at block borders, just inside and just outside the window, in prompts and in
decoding, keys in one slice and in several; the short convolution without bias or activation over a range of a wider
projection's columns, across steps shorter than its taps and a reused slot; sigmoid routing with a correction, groups
scored by their two best and plain weights; the clamped experts' unit with the routing weights applied; the token side
gate, the stream's narrowing and the sigmoid gates; latent attention with directly projected queries in a wider
projection, neighbours rotated with scaled cosines, and head gates; the exact gelu on rows of any length."""
from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def scrambled_pools(lengths, kv_heads, dim, vdim, dtype, seed, spare=3):
    """Key and value pools filled with large numbers where nothing is written, and a table whose rows name blocks in a
    shuffled order."""
    g = torch.Generator().manual_seed(seed)
    need = [-(-n // 64) for n in lengths]
    total = sum(need) + spare
    order = torch.randperm(total, generator=g).tolist()
    table = torch.full((len(lengths), max(need)), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(need):
        for i in range(n):
            table[b, i] = order[at]
            at += 1
    k_pool = torch.full((total, kv_heads, 64, dim), 300.0, dtype=dtype, device=DEV)
    v_pool = torch.full((total, kv_heads, vdim, 64), 300.0, dtype=dtype, device=DEV)
    return k_pool, v_pool, table.to(DEV)


def fill_pools(k_pool, v_pool, table, b, keys, values):
    """keys [n, kv_heads, dim], values [n, kv_heads, vdim] (float64) into sequence b's cache; returns what the cache holds."""
    ks, vs = keys.to(k_pool.dtype), values.to(v_pool.dtype)
    for pos in range(keys.shape[0]):
        block = int(table[b, pos // 64])
        k_pool[block, :, pos % 64] = ks[pos].to(DEV)
        v_pool[block, :, :, pos % 64] = vs[pos].to(DEV)
    return ks.double(), vs.double()


def attention_plain(q, keys, values, pos, heads, kv_heads, scale, window, cap, slopes, gate, per_head):
    """One query token q [heads, dim] at position pos over keys [n, kv_heads, dim], values [n, kv_heads, vdim]."""
    lo = 0 if window <= 0 else max(0, pos - window + 1)
    out = []
    for h in range(heads):
        g = h // (heads // kv_heads)
        s = (keys[lo:pos + 1, g] @ q[h]) * scale
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        if slopes is not None:
            s = s - slopes[h] * (pos - torch.arange(lo, pos + 1, dtype=torch.float64))
        o = torch.softmax(s, dim=0) @ values[lo:pos + 1, g]
        if gate is not None:
            z = gate[h] if per_head else gate[h * o.numel():(h + 1) * o.numel()]
            o = o / (1.0 + torch.exp(-z))
        out.append(o)
    return torch.cat(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,window,cap,slope,gate", [
    (4, 2, 64, 64, 80, 35.0, True, "elementwise"), (3, 3, 16, 24, 21, 30.0, True, "elementwise"), (6, 2, 48, 8, 0, 0.0, True, None),
    (2, 2, 20, 36, 64, 5.0, False, "head"), (8, 2, 128, 128, 130, 40.0, True, "elementwise"), (1, 1, 8, 8, 1, 0.0, True, "head"),
    (5, 5, 32, 32, 65, 20.0, True, None), (6, 2, 64, 64, 100, 30.0, True, "elementwise"), (14, 2, 128, 128, 0, 45.0, True, "head")])
def test_attention_marked_keys(dtype, heads, kv_heads, dim, vdim, window, cap, slope, gate):
    """Sequences of unequal lengths, prompts and decoding, through a scrambled table.  In every sequence one key is lined up
    with the last query of head 0: without a window far back or at a block border; with a window just inside the last token's
    window for two sequences and just outside it for the other two (the last head: its slope is the gentlest).  Dropping the key from the plain computation moves the
    output where it is visible.  The gate is a range of a wider projection's columns."""
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(heads * 100 + dim + window)
    scale = 0.3 / math.sqrt(dim)
    totals, new = [300, 410, 70, 131], [5, 1, 70, 1]
    slopes = torch.pow(2.0, -8.0 * torch.arange(1, heads + 1, dtype=torch.float64) / heads) if slope else None
    slopes_d = None if slopes is None else slopes.float().to(DEV)
    slopes = None if slopes is None else slopes_d.double().cpu()
    k_pool, v_pool, table = scrambled_pools(totals, kv_heads, dim, vdim, dtype, 11)
    cached, queries = [], []
    for b, n in enumerate(totals):
        keys = torch.randn(n, kv_heads, dim, generator=g, dtype=torch.float64)
        values = torch.randn(n, kv_heads, vdim, generator=g, dtype=torch.float64)
        q = torch.randn(new[b], heads, dim, generator=g, dtype=torch.float64).to(dtype).double()
        last = n - 1
        marked = [3, 63, 64, 127][b] if window <= 0 else (last - window + 1 if b in (0, 3) else last - window)
        marked = min(max(marked, 0), last)
        # a scaled score of about 30 for the last query of the last head, whose slope is the gentlest: a far key still shows
        keys[marked, kv_heads - 1] = q[-1, heads - 1] / q[-1, heads - 1].norm() ** 2 * 30.0 / scale
        cached.append(fill_pools(k_pool, v_pool, table, b, keys, values))
        queries.append(q)
    q_all = torch.cat(queries)
    tokens = q_all.shape[0]
    gate_cols = 0 if gate is None else (heads if gate == "head" else heads * vdim)
    wide = torch.randn(2, tokens, 7 + gate_cols + 3, generator=g, dtype=torch.float64).float()
    gate_view = wide.to(DEV)[:, :, 7:7 + gate_cols] if gate else None
    gate_sum = wide.double().sum(0)[:, 7:7 + gate_cols] if gate else None
    cu = [0]
    for n in new:
        cu.append(cu[-1] + n)
    before = [t - n for t, n in zip(totals, new)]
    want = []
    for b in range(len(totals)):
        for i in range(new[b]):
            row = cu[b] + i
            want.append(attention_plain(queries[b][i], cached[b][0], cached[b][1], before[b] + i, heads, kv_heads, scale, window, cap, slopes,
                                        None if gate is None else gate_sum[row], gate == "head"))
    want = torch.stack(want)
    if window != 1:
        shadow = cached[0][0].clone()
        shadow[3 if window <= 0 else totals[0] - window] = 0.0
        moved = attention_plain(queries[0][-1], shadow, cached[0][1], totals[0] - 1, heads, kv_heads, scale, window, cap, slopes,
                                None if gate is None else gate_sum[cu[1] - 1], gate == "head")
        assert float((moved - want[cu[1] - 1]).abs().max()) > 0.02
    for splits in (1, 3):
        pick = [b for b in range(len(new)) if new[b] == 1] if splits > 1 else list(range(len(new)))
        rows_of = [r for b in pick for r in range(cu[b], cu[b + 1])]
        q_step = q_all[rows_of].reshape(len(rows_of), heads * dim).to(dtype).to(DEV)
        cu_step = [0]
        for b in pick:
            cu_step.append(cu_step[-1] + new[b])
        out = torch.zeros(len(rows_of), heads * vdim, dtype=dtype, device=DEV)
        part_acc = torch.zeros(len(rows_of) * heads * splits * vdim, dtype=torch.float32, device=DEV)
        part_ml = torch.zeros(len(rows_of) * heads * splits * 2, dtype=torch.float32, device=DEV)
        word = status()
        step_gate = None
        if gate:
            step_gate = wide[:, rows_of].contiguous().to(DEV)[:, :, 7:7 + gate_cols]
        api.attention(q_step, k_pool, v_pool, table[pick].contiguous(), i32(cu_step), i32([before[b] for b in pick]), len(pick), len(rows_of),
                      heads, kv_heads, dim, scale, window, splits, out, part_acc, part_ml, word, value_dim=vdim, softcap=cap, slopes=slopes_d,
                      gate=step_gate, gate_per_head=gate == "head")
        assert int(word.item()) == 0
        err = float((out.double().cpu() - want[rows_of]).abs().max())
        bound = (2e-5 if dtype == torch.float32 else 0.03) * max(1.0, float(want.abs().max()))
        assert err <= bound, f"splits {splits}: {err}"
    # the tensor-core prompt kernel shapes its scores the same way
    if dtype == torch.bfloat16 and dim == vdim and api.attention_tcgen05_supports(dtype, heads, kv_heads, dim):
        out = torch.zeros(tokens, heads * vdim, dtype=dtype, device=DEV)
        word = status()
        api.attention_tcgen05(q_all.reshape(tokens, heads * dim).to(dtype).to(DEV), k_pool, v_pool, table, i32(cu), i32(before), len(new), tokens, heads,
                              kv_heads, dim, scale, window, out, word, softcap=cap, slopes=slopes_d, gate=gate_view, gate_per_head=gate == "head")
        assert int(word.item()) == 0
        err = float((out.double().cpu() - want).abs().max())
        assert err <= 0.04 * max(1.0, float(want.abs().max())), f"tcgen05: {err}"
    # the tensor-core decode kernel's shaped instances, keys in one slice, in a cluster's slices and in more than a cluster holds
    if dtype == torch.bfloat16 and dim == vdim and api.attention_mma_supports(dtype, heads, kv_heads, dim):
        pick = [b for b in range(len(new)) if new[b] == 1]
        rows_of = [cu[b] for b in pick]
        for splits in (1, 2, 11):
            out = torch.zeros(len(pick), heads * vdim, dtype=dtype, device=DEV)
            part_acc = torch.zeros(len(pick) * heads * splits * vdim, dtype=torch.float32, device=DEV)
            part_ml = torch.zeros(len(pick) * heads * splits * 2, dtype=torch.float32, device=DEV)
            word = status()
            api.attention_mma(q_all[rows_of].reshape(len(pick), heads * dim).to(dtype).to(DEV), k_pool, v_pool, table[pick].contiguous(), i32(list(range(len(pick) + 1))),
                              i32([before[b] for b in pick]), len(pick), len(pick), heads, kv_heads, dim, scale, window, splits, out, part_acc, part_ml, word,
                              one_token_each=True, softcap=cap, slopes=slopes_d)
            if gate:
                api.sigmoid_gate(out, wide[:, rows_of].contiguous().to(DEV)[:, :, 7:7 + gate_cols], vdim if gate == "head" else 0)
            assert int(word.item()) == 0
            err = float((out.double().cpu() - want[rows_of]).abs().max())
            assert err <= 0.04 * max(1.0, float(want.abs().max())), f"decode on tensor cores, {splits} slices: {err}"


@pytest.mark.parametrize("taps", [1, 2, 3, 4, 6])
def test_convolution_over_a_range_of_columns(taps):
    """No bias, no activation, the first channels of a wider projection in two slices; two sequences in steps of unequal
    sizes, some shorter than the taps; then the slot of the first is used again from zeros."""
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(taps)
    channels, extra, slots = 40, 9, 3
    weight = torch.randn(channels, taps, generator=g, dtype=torch.float64).float()
    state = torch.zeros(slots, taps - 1, channels, dtype=torch.float32, device=DEV)

    def plain(u):
        padded = torch.cat([torch.zeros(taps - 1, channels, dtype=torch.float64), u])
        return sum(padded[j:j + u.shape[0]] * weight.double()[:, j] for j in range(taps))

    def run(sequences):
        """sequences: slot -> float64 inputs [n, channels]; steps of unequal sizes, both sequences in every step they have tokens for"""
        cuts = {slot: list(c) for slot, c in zip(sequences, ([1, 2, 1, 7, 1, 30], [5, 1, 1, 1, 40]))}
        at = {slot: 0 for slot in sequences}
        got = {slot: [] for slot in sequences}
        while any(cuts.values()):
            live = [slot for slot in sequences if cuts[slot]]
            counts = [min(cuts[slot].pop(0), sequences[slot].shape[0] - at[slot]) for slot in live]
            rows = torch.cat([sequences[slot][at[slot]: at[slot] + n] for slot, n in zip(live, counts)])
            proj = torch.zeros(2, rows.shape[0], channels + extra, dtype=torch.float32)
            proj[0, :, :channels] = rows.float() * 0.25
            proj[1, :, :channels] = rows.float() * 0.75
            proj[:, :, channels:] = 1e6
            cu = [0]
            for n in counts:
                cu.append(cu[-1] + n)
            out = torch.zeros(rows.shape[0], channels, dtype=torch.float32, device=DEV)
            api.causal_conv(proj.to(DEV), 0, channels, weight.to(DEV), None, False, state, out, i32(cu), i32(live), len(live), rows.shape[0],
                            all(n == 1 for n in counts))
            for i, (slot, n) in enumerate(zip(live, counts)):
                got[slot].append(out[cu[i]: cu[i + 1]].double().cpu())
                at[slot] += n
        return {slot: torch.cat(parts) for slot, parts in got.items()}

    first = {2: torch.randn(42, channels, generator=g, dtype=torch.float64).float().double(), 0: torch.randn(48, channels, generator=g, dtype=torch.float64).float().double()}
    got = run(first)
    for slot, u in first.items():
        assert float((got[slot] - plain(u)).abs().max()) < 1e-4 * float(plain(u).abs().max()), (taps, slot)
    state[2].zero_()                                   # what handing the slot out again does
    again = {2: torch.randn(42, channels, generator=g, dtype=torch.float64).float().double(), 1: torch.randn(48, channels, generator=g, dtype=torch.float64).float().double()}
    got = run(again)
    for slot, u in again.items():
        assert float((got[slot] - plain(u)).abs().max()) < 1e-4 * float(plain(u).abs().max()), (taps, slot, "again")


def route_plain(z, correction, top, groups, keep, sigmoid, top2, plain_weights):
    E = z.numel()
    s = 1.0 / (1.0 + torch.exp(-z)) if sigmoid else torch.softmax(z, dim=0)
    c = s + (correction if correction is not None else 0.0)
    size = E // groups
    if top2:
        group = torch.topk(c.reshape(groups, size), min(2, size), dim=1).values.sum(dim=1)
    else:
        group = c.reshape(groups, size).max(dim=1).values
    kept = sorted(range(groups), key=lambda i: (-float(group[i]), i))[:keep]
    allowed = [e for e in range(E) if e // size in kept]
    chosen = sorted(allowed, key=lambda e: (-float(c[e]), e))[:top]
    w = torch.stack([s[e] for e in chosen])
    return chosen, (w if plain_weights else w / (w.sum() + 1e-20))


@pytest.mark.parametrize("experts,top,groups,keep,extra", [(16, 4, 4, 2, 1), (6, 2, 3, 2, 1), (8, 3, 4, 2, 0), (5, 5, 1, 1, 1), (4, 1, 4, 2, 2),
                                                          (64, 6, 8, 4, 0), (12, 4, 12, 5, 1), (9, 2, 3, 3, 0)])
@pytest.mark.parametrize("sigmoid,top2,plain_weights,corrected", [(True, True, True, True), (True, False, False, False), (False, True, True, True),
                                                                   (False, False, False, False)])
def test_routing_options(experts, top, groups, keep, extra, sigmoid, top2, plain_weights, corrected):
    """The routing alone (logits in two slices) and with the router's product in front, against a plain top-k; the
    correction is large enough to make choice scores negative and to change the choice; the always-on gates ride behind."""
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(experts * 10 + top)
    tokens, hidden = 37, 48
    x = torch.randn(tokens, hidden, generator=g, dtype=torch.float64).float()
    w = (torch.randn(experts + extra, hidden, generator=g, dtype=torch.float64) * 0.4).float()
    correction = (torch.randn(experts, generator=g, dtype=torch.float64) * 0.8 - 1.0).float() if corrected else None
    z = x.double() @ w.double().T
    options = {"score": "sigmoid" if sigmoid else "softmax", "correction": None if correction is None else correction.to(DEV),
               "group_score": "top2" if top2 else "max", "renormalize": not plain_weights, "extra": extra}
    halves = torch.stack([z * 0.3, z * 0.7]).float().to(DEV).contiguous()
    for form in ("logits", "rows"):
        gates = torch.full((tokens, experts + extra), 7.0, dtype=torch.float32, device=DEV)
        chosen = torch.full((tokens, top), -5, dtype=torch.int32, device=DEV)
        weights = torch.full((tokens, top), 7.0, dtype=torch.float32, device=DEV)
        if form == "logits":
            api.route_topk(halves, top, groups, keep, gates, chosen, weights, **options)
        else:
            api.route_rows(x.to(DEV), w.to(DEV), top, groups, keep, gates, chosen, weights, **options)
        torch.cuda.synchronize()
        for t in range(tokens):
            want, want_w = route_plain(z[t, :experts], None if correction is None else correction.double(), top, groups, keep, sigmoid, top2, plain_weights)
            got = [int(e) for e in chosen[t].cpu() if int(e) >= 0]
            # a near tie may fall the other way in float32; then the sets differ by experts whose choice scores nearly agree
            if got != want:
                s = 1.0 / (1.0 + torch.exp(-z[t, :experts])) if sigmoid else torch.softmax(z[t, :experts], dim=0)
                c = s + (correction.double() if correction is not None else 0.0)
                assert sorted(got) == sorted(want) or abs(float(c[list(set(got) ^ set(want))].max() - c[list(set(got) ^ set(want))].min())) < 1e-5, (form, t, got, want)
                continue
            assert torch.allclose(weights[t, :len(want)].double().cpu(), want_w, rtol=2e-5, atol=1e-7), (form, t)
            dense = torch.zeros(experts, dtype=torch.float64)
            dense[want] = want_w
            assert torch.allclose(gates[t, :experts].double().cpu(), dense, rtol=2e-5, atol=1e-7), (form, t)
            if extra:
                assert torch.allclose(gates[t, experts:].double().cpu(), 1.0 / (1.0 + torch.exp(-z[t, experts:])), rtol=2e-5), (form, t)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,width,shared,limit,shared_limit,gated", [(4, 24, 16, 1.25, 2.5, True), (3, 10, 0, 0.5, 0.0, False), (6, 8, 12, 0.0, 0.75, False),
                                                                           (1, 33, 7, 7.0, 7.0, True)])
def test_expert_activation(dtype, experts, width, shared, limit, shared_limit, gated):
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(experts + width)
    tokens, cols = 19, experts * width + shared
    gate_up = (torch.randn(3, tokens, 2 * cols, generator=g, dtype=torch.float64) * 1.5).float()
    gates = torch.rand(tokens, experts + 1, generator=g, dtype=torch.float64).float()
    gates[:, :experts][torch.rand(tokens, experts, generator=g) < 0.5] = 0.0
    act = torch.full((tokens, cols), 9.0, dtype=dtype, device=DEV)
    api.expert_activation(gate_up.to(DEV), act, experts, width, shared, limit, shared_limit, 1.702, gates.to(DEV), gated)
    total = gate_up.double().sum(0)
    gt, up = total[:, :cols], total[:, cols:]
    want = torch.zeros(tokens, cols, dtype=torch.float64)
    for c in range(cols):
        routed = c < experts * width
        lim = limit if routed else shared_limit
        a, u = gt[:, c], up[:, c]
        if lim > 0:
            a, u = torch.clamp(a, max=lim), torch.clamp(u, -lim, lim)
        weight = gates[:, c // width].double() if routed else (gates[:, experts].double() if gated else 1.0)
        want[:, c] = a / (1.0 + torch.exp(-1.702 * a)) * (u + 1.0) * weight
    bound = 1e-5 if dtype == torch.float32 else 0.01
    assert float((act.double().cpu() - want).abs().max()) <= bound * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_side_gate_stream_and_gates(dtype):
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(5)
    tokens, hidden, dim, vocab, layers = 23, 50, 6, 31, 4
    bound = 1e-6 if dtype == torch.float32 else 0.01
    # the stream takes a delta in two slices and is handed on narrowed; without a delta it is only narrowed
    residual = torch.randn(tokens, hidden, generator=g, dtype=torch.float64).float()
    delta = torch.randn(2, tokens, hidden, generator=g, dtype=torch.float64).float()
    stream, out = residual.clone().to(DEV), torch.zeros(tokens, hidden, dtype=dtype, device=DEV)
    api.add_narrow(stream, delta.to(DEV), out)
    want = residual.double() + delta.double().sum(0)
    assert float((stream.double().cpu() - want).abs().max()) < 1e-6 and float((out.double().cpu() - want).abs().max()) <= bound * 5
    api.add_narrow(stream, None, out)
    assert float((stream.double().cpu() - want).abs().max()) < 1e-6 and float((out.double().cpu() - want).abs().max()) <= bound * 5
    # the gate times the layer's slice of the token's row
    table = torch.randn(vocab, layers * dim, generator=g, dtype=torch.float64).to(dtype)
    ids = torch.randint(0, vocab, (tokens,), generator=g)
    x = torch.randn(2, tokens, dim, generator=g, dtype=torch.float64).float()
    for layer in (0, 3):
        gated = torch.zeros(tokens, dim, dtype=dtype, device=DEV)
        word = status()
        api.token_side_gate(x.to(DEV), table.to(DEV), layer * dim, ids.to(torch.int32).to(DEV), gated, word)
        z = x.double().sum(0)
        want = 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3))) * table.double()[ids][:, layer * dim:(layer + 1) * dim]
        assert int(word.item()) == 0 and float((gated.double().cpu() - want).abs().max()) <= bound * 5
    word = status()
    api.token_side_gate(x.to(DEV), table.to(DEV), 0, torch.full((tokens,), vocab, dtype=torch.int32, device=DEV), gated, word)
    assert int(word.item()) == api.STATUS_BAD_TOKEN and float(gated.abs().max()) == 0.0
    # sigmoid gates in place, one number per output number and one per head, out of a wider projection
    heads, vdim = 3, 8
    y = torch.randn(tokens, heads * vdim, generator=g, dtype=torch.float64).to(dtype)
    wide = torch.randn(2, tokens, 5 + heads * vdim + heads, generator=g, dtype=torch.float64).float()
    got = y.clone().to(DEV)
    api.sigmoid_gate(got, wide.to(DEV)[:, :, 5:5 + heads * vdim])
    want = y.double() / (1.0 + torch.exp(-wide.double().sum(0)[:, 5:5 + heads * vdim]))
    assert float((got.double().cpu() - want).abs().max()) <= bound * 5
    got = y.clone().to(DEV)
    api.sigmoid_gate(got, wide.to(DEV)[:, :, 5 + heads * vdim:], vdim)
    want = y.double() / (1.0 + torch.exp(-wide.double().sum(0)[:, 5 + heads * vdim:].repeat_interleave(vdim, dim=1)))
    assert float((got.double().cpu() - want).abs().max()) <= bound * 5


@pytest.mark.parametrize("inter", [8, 102, 7])
def test_exact_gelu_on_rows_of_any_length(inter):
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(inter)
    x = (torch.randn(2, 13, inter, generator=g, dtype=torch.float64) * 2.0).float()
    act = torch.full((13, inter), 9.0, dtype=torch.float32, device=DEV)
    api.activation(x.to(DEV), act, "gelu")
    z = x.double().sum(0)
    want = 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))
    assert float((act.double().cpu() - want).abs().max()) < 2e-6


def rotate_pairs_plain(x, pos, inv_freq, dims, factor):
    """x [..., n] float64 at one position: neighbours of the first ``dims`` numbers paired, cosines and sines times ``factor``."""
    angle = (torch.tensor(float(pos), dtype=torch.float32) * inv_freq.cpu().float()[:dims // 2]).double()
    cos, sin = angle.cos() * factor, angle.sin() * factor
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([u * cos - v * sin, v * cos + u * sin], dim=-1).reshape(*x.shape[:-1], dims)
    return torch.cat([turned, x[..., dims:]], dim=-1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,rot,vdim,rank,gated", [(4, 48, 16, 64, 80, True), (2, 24, 8, 16, 40, True), (1, 48, 16, 8, 24, False), (3, 20, 6, 12, 18, True),
                                                          (16, 32, 32, 64, 48, True)])
def test_latent_attention_with_direct_queries(dtype, heads, dim, rot, vdim, rank, gated):
    """One wide projection [kv latent | key part | queries | head gates] in two slices through the prepare kernel (no query
    latent) and the attention kernels: cache rows, rotation of neighbours with scaled cosines, head gates; prompts in two
    portions and decoding, with a far key lined up with the last query."""
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(heads * 7 + rank)
    scale, eps, factor = 0.2, 1e-5, 1.0693
    inv_freq = (500.0 ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot)).float().to(DEV)
    lengths, cuts = [150, 70], [(90, 59, 1), (69, 1)]
    front, q_cols = rank + rot, heads * (dim + rot)
    cols = front + q_cols + heads
    norm = (1.0 + 0.1 * torch.randn(rank, generator=g, dtype=torch.float64)).float()
    w_key = (torch.randn(heads * dim, rank, generator=g, dtype=torch.float64) * 0.3).to(dtype)
    w_value = (torch.randn(heads * vdim, rank, generator=g, dtype=torch.float64) * 0.3).to(dtype)
    pool = torch.full((8, 1, 64, front), 300.0, dtype=dtype, device=DEV)
    table = i32([[5, 2, 7], [1, 4, -1]])
    rows = [torch.randn(n, cols, generator=g, dtype=torch.float64).float().double() for n in lengths]
    for b, n in enumerate(lengths):                     # the last query's head 0 finds position 3
        c = rows[b][3, :rank]
        c = c / torch.sqrt((c * c).mean() + eps) * norm.double()
        c = c.to(dtype).double()
        a = w_key.double()[:dim].T @ rows[b][n - 1, front:front + dim]
        rows[b][n - 1, front:front + dim] *= 20.0 / (scale * float(a @ c))
    want, got = [[] for _ in lengths], [[] for _ in lengths]
    cached = []
    for b, n in enumerate(lengths):
        c = rows[b][:, :rank]
        c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * norm.double()
        kr = torch.stack([rotate_pairs_plain(rows[b][p, rank:front], p, inv_freq, rot, factor) for p in range(n)])
        cached.append(torch.cat([c, kr], dim=1).to(dtype).double())
        for p in range(n):
            q = rows[b][p, front:front + q_cols].reshape(heads, dim + rot)
            out = []
            for h in range(heads):
                k_plain = cached[b][:p + 1, :rank] @ w_key.double()[h * dim:(h + 1) * dim].T
                s = (k_plain @ q[h, :dim] + cached[b][:p + 1, rank:] @ rotate_pairs_plain(q[h, dim:], p, inv_freq, rot, factor)) * scale
                o = (torch.softmax(s, dim=0) @ cached[b][:p + 1, :rank]) @ w_value.double()[h * vdim:(h + 1) * vdim].T
                if gated:
                    o = o / (1.0 + torch.exp(-rows[b][p, front + q_cols + h]))
                out.append(o)
            want[b].append(torch.cat(out))
    at = [0, 0]
    for step in range(3):
        live = [b for b in range(2) if step < len(cuts[b])]
        counts = [cuts[b][step] for b in live]
        packed = torch.cat([rows[b][at[b]: at[b] + n] for b, n in zip(live, counts)])
        wide = torch.stack([packed * 0.25, packed * 0.75]).float().to(DEV).contiguous()
        cu = [0]
        for n in counts:
            cu.append(cu[-1] + n)
        tokens = packed.shape[0]
        word = status()
        step_table = table[live].contiguous()
        api.latent_prepare(wide[:, :, :front], 0, rank, rot, None, norm.to(DEV), eps, inv_freq, rot, None, pool, step_table, i32(cu), i32([at[b] for b in live]),
                           len(live), tokens, word, interleaved=True, rot_scale=factor)
        decode = all(n == 1 for n in counts)
        for splits in ((1, 2) if decode else (1,)):
            out = torch.zeros(tokens, heads * vdim, dtype=dtype, device=DEV)
            absorbed = torch.zeros(tokens * heads * front, dtype=torch.float32, device=DEV)
            part_acc = torch.zeros(tokens * heads * splits * rank, dtype=torch.float32, device=DEV)
            part_ml = torch.zeros(tokens * heads * splits * 2, dtype=torch.float32, device=DEV)
            api.latent_attention(wide[:, :, front:front + q_cols], w_key.to(DEV), w_value.to(DEV), pool, step_table, i32(cu), i32([at[b] for b in live]),
                                 len(live), tokens, heads, dim, rot, vdim, rank, inv_freq, rot, scale, 0, splits, out, absorbed, part_acc, part_ml, word,
                                 interleaved=True, rot_scale=factor, head_gate=wide[:, :, front + q_cols:] if gated else None)
            assert int(word.item()) == 0
            for i, (b, n) in enumerate(zip(live, counts)):
                expect = torch.stack(want[b][at[b]: at[b] + n])
                err = float((out[cu[i]: cu[i + 1]].double().cpu() - expect).abs().max())
                assert err <= (3e-5 if dtype == torch.float32 else 0.04) * max(1.0, float(expect.abs().max())), (step, b, splits, err)
        # the expanded form's queries: the same rotation, narrowed
        queries = torch.zeros(tokens, q_cols, dtype=dtype, device=DEV)
        api.latent_queries(wide[:, :, front:front + q_cols], heads, dim, rot, inv_freq, rot, i32(cu), i32([at[b] for b in live]), len(live), tokens, queries,
                           interleaved=True, rot_scale=factor)
        row = 0
        for b, n in zip(live, counts):
            for p in range(at[b], at[b] + n):
                q = rows[b][p, front:front + q_cols].reshape(heads, dim + rot)
                expect = torch.cat([q[:, :dim], torch.stack([rotate_pairs_plain(q[h, dim:], p, inv_freq, rot, factor) for h in range(heads)])], dim=1).reshape(-1)
                assert float((queries[row].double().cpu() - expect).abs().max()) <= (1e-5 if dtype == torch.float32 else 0.02) * max(1.0, float(expect.abs().max()))
                row += 1
        for b, n in zip(live, counts):
            at[b] += n
    # the cache holds the normed latents and the rotated key parts, and nothing else was written
    for b, n in enumerate(lengths):
        for p in (0, 3, 63, 64, n - 1):
            held = pool[int(table[b, p // 64]), 0, p % 64].double().cpu()
            assert float((held - cached[b][p]).abs().max()) <= (1e-5 if dtype == torch.float32 else 0.02) * max(1.0, float(cached[b][p].abs().max()))
    assert float(pool[0].min()) == 300.0 and float(pool[int(table[1, 1]), 0, lengths[1] % 64:].min()) == 300.0


@pytest.mark.parametrize("tokens", [8, 130, 700])
def test_clamped_unit_as_the_gated_products_epilogue(tokens):
    """The tensor-core gated product with the clamped unit as its epilogue and the column scaling behind it, against the
    plain formula: routed experts' columns with one limit, the shared expert's behind them with another and its own gate."""
    from thintensor_b200.kernels import api

    g = torch.Generator().manual_seed(tokens)
    k, experts, width, shared = 64, 5, 24, 40
    cols = experts * width + shared
    x = torch.randn(tokens, k, generator=g, dtype=torch.float64).to(torch.bfloat16)
    w = (torch.randn(2 * cols, k, generator=g, dtype=torch.float64) * 0.3).to(torch.bfloat16)
    gates = torch.rand(tokens, experts + 1, generator=g, dtype=torch.float64).float()
    gates[:, :experts][torch.rand(tokens, experts, generator=g) < 0.5] = 0.0
    act = torch.full((tokens, cols), 9.0, dtype=torch.bfloat16, device=DEV)
    word = status()
    api.gemm_tcgen05_clamped(x.to(DEV), w.to(DEV), act, word, 1.0, 2.5, experts * width, 1.702)
    api.scale_expert_columns(act, width, gates.to(DEV), experts, shared)
    assert int(word.item()) == 0
    both = x.double() @ w.double().T
    gt, up = both[:, :cols], both[:, cols:]
    limit = torch.cat([torch.full((experts * width,), 1.0), torch.full((shared,), 2.5)]).double()
    a, u = torch.minimum(gt, limit), torch.maximum(torch.minimum(up, limit), -limit)
    weight = torch.cat([gates[:, :experts].double().repeat_interleave(width, dim=1), gates[:, experts:].double().expand(tokens, shared)], dim=1)
    want = a / (1.0 + torch.exp(-1.702 * a)) * (u + 1.0) * weight
    assert float((act.double().cpu() - want).abs().max()) <= 0.02 * max(1.0, float(want.abs().max()))
