"""Each mechanism of the Sogidra layers alone: the kernel against the plain implementation's function for it, at sizes
of its own, with inputs made so that a fault shows: a far key that dominates, keys just inside and just outside a
window, a block of tokens that has just become visible as its mean and one that has not yet, tokens that are in neither,
cache blocks handed out in a scrambled order, sequences that continue from a cache other steps filled."""
from __future__ import annotations

import math

import pytest
import torch

import plain_sogidra as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"
BLOCK = 64


def randn(*shape, seed, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float32) * scale


def slices(x: torch.Tensor, n: int, seed: int) -> torch.Tensor:
    """x as n partial sums [n, ...] that add up to it (up to float32 rounding of the last one)."""
    parts = [randn(*x.shape, seed=seed + i) for i in range(n - 1)]
    return torch.stack(parts + [x - sum(parts)] if parts else [x])


def ints(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def cu_of(news):
    return ints([0] + torch.tensor(news).cumsum(0).tolist())


class Pools:
    """A key pool and a transposed value pool with a block table whose rows name blocks in a scrambled order."""

    def __init__(self, sequences, most_tokens, kv_heads, key_dim, value_dim, dtype, seed):
        width = -(-most_tokens // BLOCK)
        self.blocks = sequences * width + 3
        order = torch.randperm(self.blocks, generator=torch.Generator().manual_seed(seed)).tolist()
        self.table = ints([[order[b * width + i] for i in range(width)] for b in range(sequences)])
        # not zeros: a kernel that reads an entry nobody wrote meets large numbers
        self.k = torch.full((self.blocks, kv_heads, BLOCK, key_dim), 50.0, dtype=dtype, device=DEV)
        self.v = torch.full((self.blocks, kv_heads, value_dim, BLOCK), -50.0, dtype=dtype, device=DEV)

    def put(self, b, position, keys, values):
        """keys [kv_heads, key_dim], values [kv_heads, value_dim] of one token (or entry)."""
        block = int(self.table[b, position // BLOCK])
        self.k[block, :, position % BLOCK] = keys.to(self.k.dtype).to(DEV)
        self.v[block, :, :, position % BLOCK] = values.to(self.v.dtype).to(DEV)

    def key(self, b, position):
        return self.k[int(self.table[b, position // BLOCK]), :, position % BLOCK].double().cpu()

    def value(self, b, position):
        return self.v[int(self.table[b, position // BLOCK]), :, :, position % BLOCK].double().cpu()


# ---------------------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("hidden", [72, 192, 333, 4100])
@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_norm_chain(hidden, splits, out_dtype):
    """The norm of a sublayer's output on its way into the stream, the keeping of results, their weighted sum and the
    norm that follows, in every combination a layer uses; and wanted rows only, which must write nothing else."""
    from thintensor_b200.kernels import api

    rows, count, eps = 6, 4, 1e-5
    residual = randn(rows, hidden, seed=1, scale=3.0)
    delta = randn(rows, hidden, seed=2, scale=20.0)           # far larger than the stream: a forgotten norm shows
    post_w, w = randn(hidden, seed=3, scale=0.2), randn(hidden, seed=4, scale=0.2)
    earlier = randn(count, rows, hidden, seed=5, scale=2.0)
    depth_w = randn(count, seed=6) + 0.5
    tol = 3e-5 if out_dtype == torch.float32 else 2e-2

    def close(got, want, what):
        assert float((got.double().cpu() - want).abs().max()) <= tol * max(1.0, float(want.abs().max())), what

    for use_post in (False, True):
        for index in (None, 0, 2, 3):
            for pick in (None, [4, 0, 4]):
                res = residual.clone().to(DEV)
                kept = earlier.clone().to(DEV)
                out = torch.empty(len(pick) if pick else rows, hidden, dtype=out_dtype, device=DEV)
                mixes = index is not None and index > 0
                api.add_rmsnorm_chain(res, slices(delta, splits, 10).to(DEV), post_w.to(DEV) if use_post else None, 1.0, eps,
                                      kept if index is not None else None, index or 0, depth_w.to(DEV) if mixes else None, w.to(DEV), 1.0,
                                      eps, out, ints(pick) if pick else None)
                v = delta.double()
                if use_post:
                    v = plain.zero_centred_norm(v, post_w.double(), eps)
                result = residual.double() + v
                x = result
                if mixes:
                    x = sum(float(depth_w[j]) * earlier[j].double() for j in range(index)) + float(depth_w[index]) * result
                want = plain.zero_centred_norm(x, w.double(), eps)
                what = f"post {use_post} index {index} rows {pick}"
                if pick:
                    close(out, want[pick], what)
                    assert torch.equal(res.cpu(), residual) and torch.equal(kept.cpu(), earlier), what
                else:
                    close(out, want, what)
                    assert float((res.double().cpu() - x).abs().max()) <= 3e-5 * max(1.0, float(x.abs().max())), what
                    if index is not None:
                        assert float((kept[index].double().cpu() - result).abs().max()) <= 3e-5 * float(result.abs().max()), what
                        others = [j for j in range(count) if j != index]
                        assert torch.equal(kept[others].cpu(), earlier[others]), what


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_xielu_and_the_other_activations(out_dtype):
    from thintensor_b200.kernels import api

    tokens, inter = 5, 76
    x = randn(3, tokens, inter, seed=7, scale=3.0)
    x[0, 0, :8] = torch.tensor([0.0, 1e-4, -1e-4, 30.0, -30.0, -1e-3, 0.5, -0.5]) - x[1:, 0, :8].sum(0)    # around zero and far out
    z = x.double().sum(0)
    p, q = 0.7, -1.3
    act = torch.empty(tokens, inter, dtype=out_dtype, device=DEV)
    api.activation(x.to(DEV), act, "xielu", plain.softplus(p), 0.5 + plain.softplus(q))
    want = plain.xielu(z, p, q)
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    assert float(((act.double().cpu() - want).abs() / (1.0 + want.abs())).max()) <= tol
    api.activation(x.to(DEV), act, "gelu_tanh")
    want = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
    assert float(((act.double().cpu() - want).abs() / (1.0 + want.abs())).max()) <= tol


@pytest.mark.parametrize("stored", [torch.float32, torch.bfloat16])
def test_embedding_with_learned_positions(stored):
    """Sequences that start at position 0 beside ones that continue; a position beyond the table raises the status word."""
    from thintensor_b200.kernels import api

    vocab, hidden, most = 50, 72, 40
    table, positions = randn(vocab, hidden, seed=8).to(stored), randn(most, hidden, seed=9).to(stored)
    news, before = [3, 1, 5], [0, 39, 17]
    tokens = [7, 0, 49, 3, 11, 12, 13, 14, 15]
    residual = torch.empty(len(tokens), hidden, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    api.embed_position_gather(table.to(DEV), positions.to(DEV), ints(tokens), cu_of(news), ints(before), 3, residual, 1.0, status)
    where = [b + i for n, b in zip(news, before) for i in range(n)]
    want = table.double()[tokens] + positions.double()[where]
    assert float((residual.double().cpu() - want).abs().max()) <= 1e-6 and int(status.item()) == 0
    api.embed_position_gather(table.to(DEV), positions.to(DEV), ints(tokens), cu_of(news), ints([0, 40, 17]), 3, residual, 1.0, status)
    assert int(status.item()) == api.STATUS_BAD_TOKEN and float(residual[3].abs().max()) == 0.0


@pytest.mark.parametrize("act_dtype", [torch.float32, torch.bfloat16])
def test_queries_keys_and_values_on_their_way_to_the_cache(act_dtype):
    """The options of the general prepare kernel that these mixers use: a query gain that grows with the position (a
    period of 1 and one that the positions straddle), norms without a weight, values that are the unnormed keys."""
    from thintensor_b200.kernels import api

    heads, kv_heads, dim, vdim, eps = 3, 1, 40, 24, 1e-5
    news, before = [4, 2], [5, 62]                          # the second sequence crosses a cache block's border
    n = sum(news)
    pos = [b + i for c, b in zip(news, before) for i in range(c)]
    no_rot = torch.zeros(1, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    tol = 1e-5 if act_dtype == torch.float32 else 1e-2
    for every in (1, 6):
        proj = randn(n, heads * dim + kv_heads * (dim + vdim), seed=11)
        pools = Pools(2, 70, kv_heads, dim, vdim, act_dtype, 12)
        q = torch.empty(n, heads * dim, dtype=act_dtype, device=DEV)
        api.qk_norm_rope_append(slices(proj, 2, 13).to(DEV), None, None, 0.0, no_rot, 0, False, 1.0, q, pools.k, pools.v, pools.table,
                                cu_of(news), ints(before), 2, n, heads, kv_heads, dim, vdim, status, q_gain=(0.37, every))
        gain = torch.tensor([plain.query_temperature(p, 0.37, every) for p in pos], dtype=torch.float64)
        assert float((q.double().cpu() - proj.double()[:, : heads * dim] * gain[:, None]).abs().max()) <= tol * 8
        t = 0
        for b, (c, start) in enumerate(zip(news, before)):
            for i in range(c):
                assert float((pools.key(b, start + i)[0] - proj.double()[t, heads * dim: heads * dim + dim]).abs().max()) <= tol * 4
                assert float((pools.value(b, start + i)[0] - proj.double()[t, heads * dim + dim:]).abs().max()) <= tol * 4
                t += 1
    # unit norms, values from the unnormed keys
    proj = randn(n, (heads + kv_heads) * dim, seed=14, scale=5.0)
    pools = Pools(2, 70, kv_heads, dim, dim, act_dtype, 15)
    q = torch.empty(n, heads * dim, dtype=act_dtype, device=DEV)
    api.qk_norm_rope_append(slices(proj, 3, 16).to(DEV), None, None, eps, no_rot, 0, False, 1.0, q, pools.k, pools.v, pools.table, cu_of(news),
                            ints(before), 2, n, heads, kv_heads, dim, dim, status, unit_norm=True, value_from_keys=True)
    want_q = plain.unit_rms(proj.double()[:, : heads * dim].view(n, heads, dim), eps).view(n, -1)
    assert float((q.double().cpu() - want_q).abs().max()) <= tol * 4
    t = 0
    for b, (c, start) in enumerate(zip(news, before)):
        for i in range(c):
            raw = proj.double()[t, heads * dim:]
            assert float((pools.key(b, start + i)[0] - plain.unit_rms(raw, eps)).abs().max()) <= tol * 4
            assert float((pools.value(b, start + i)[0] - raw).abs().max()) <= tol * 25
            t += 1
    assert int(status.item()) == 0


# ---------------------------------------------------------------------------------- differential attention
def plain_differential(q, keys, values, i, h, group, dim, scale, lam, gain, eps):
    g = h // group
    maps = []
    for which in range(2):
        scores = (keys[: i + 1, g, which * dim: (which + 1) * dim] @ q[h, which * dim: (which + 1) * dim]) * scale
        maps.append(plain.softmax_row(scores) @ values[: i + 1, g])
    return plain.unit_rms(maps[0] - lam * maps[1], eps) * gain


@pytest.mark.parametrize("act_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 24, 40), (1, 1, 8, 136), (6, 2, 64, 128), (3, 3, 72, 16),
                                                  (6, 1, 48, 96), (5, 1, 32, 64), (2, 2, 128, 128)])
def test_differential_attention(heads, kv_heads, dim, vdim, act_dtype):
    """Prompt rows and decoded rows over caches of 1 to 300 tokens, whole and in slices.  In one sequence the first
    map's query is aligned with a key 250 tokens back and the second map's with a key in the next cache block, so each
    map's weight sits on a different far key and the subtraction, not an average, decides the output."""
    from thintensor_b200.kernels import api

    scale, lam, gain, eps = 0.3, 0.65, 0.45, 1e-5
    lengths = [300, 1, 65]
    # the rows asked for: each sequence's last tokens; then one token a sequence, as a decoding step brings them
    for news in ([3, 1, 2], [1, 1, 1]):
        pools = Pools(3, 320, kv_heads, 2 * dim, vdim, act_dtype, 21)
        keys = [randn(n, kv_heads, 2 * dim, seed=22 + b) for b, n in enumerate(lengths)]
        values = [randn(n, kv_heads, vdim, seed=25 + b) for b, n in enumerate(lengths)]
        q = randn(sum(news), heads, 2 * dim, seed=28)
        mark_one, mark_two = randn(dim, seed=29, scale=3.0), randn(dim, seed=30, scale=3.0)
        keys[0][49, :, :dim] = mark_one
        keys[0][70, :, dim:] = mark_two
        q[news[0] - 1, :, :dim] = mark_one * 2.0
        q[news[0] - 1, :, dim:] = mark_two * 2.0
        for b, n in enumerate(lengths):
            for p in range(n):
                pools.put(b, p, keys[b][p], values[b][p])
        before = [n - c for n, c in zip(lengths, news)]
        n_rows = sum(news)
        out = torch.empty(n_rows, heads * vdim, dtype=act_dtype, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        tol = 2e-5 if act_dtype == torch.float32 else 3e-2
        qd = q.to(act_dtype)
        for splits in (1, 2, 5):
            part_acc = torch.empty(n_rows * heads * splits * 2 * vdim, dtype=torch.float32, device=DEV)
            part_ml = torch.empty(n_rows * heads * splits * 4, dtype=torch.float32, device=DEV)
            out.fill_(7.0)
            api.differential_attention(qd.view(n_rows, -1).to(DEV), pools.k, pools.v, pools.table, cu_of(news), ints(before), 3, n_rows, heads,
                                       kv_heads, dim, vdim, scale, lam, gain, eps, splits, out, part_acc, part_ml, status)
            t = 0
            for b, (c, start) in enumerate(zip(news, before)):
                kb = torch.stack([pools.key(b, p) for p in range(lengths[b])])
                vb = torch.stack([pools.value(b, p) for p in range(lengths[b])])
                for i in range(start, start + c):
                    for h in range(heads):
                        want = plain_differential(qd[t].double(), kb, vb, i, h, heads // kv_heads, dim, scale, lam, gain, eps)
                        got = out[t].double().cpu().view(heads, vdim)[h]
                        assert float((got - want).abs().max()) <= tol, (news, splits, b, i, h)
                    t += 1
            # the marked keys carry their maps: without them the row differs by far more than the tolerance
        assert int(status.item()) == 0


# ---------------------------------------------------------------------------------- window attention with pooled blocks
def plain_pooled_row(q, keys, values, key_means, value_means, i, h, group, window, pool, scale, cap):
    g = h // group
    first, nb = max(0, i - window + 1), plain.visible_blocks(i, window, pool)
    ks = torch.cat([key_means[:nb, g], keys[first: i + 1, g]])
    vs = torch.cat([value_means[:nb, g], values[first: i + 1, g]])
    scores = (ks @ q[h]) * scale
    if cap:
        scores = cap * torch.tanh(scores / cap)
    return plain.softmax_row(scores) @ vs


@pytest.mark.parametrize("act_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,window,pool,cap", [(4, 2, 40, 21, 5, 8.0), (2, 2, 16, 70, 64, 0.0), (3, 1, 8, 1, 1, 3.0),
                                                                (2, 1, 72, 9, 30, 30.0), (4, 2, 128, 100, 16, 20.0), (2, 1, 64, 33, 8, 0.0),
                                                                (6, 3, 96, 70, 11, 15.0), (16, 1, 32, 64, 64, 5.0), (2, 2, 32, 1, 1, 0.0),
                                                                (4, 1, 64, 9, 30, 6.0), (2, 1, 128, 130, 3, 0.0)])
def test_pooled_window_attention(heads, kv_heads, dim, window, pool, cap, act_dtype):
    """The cache is filled in steps (portions of a prompt, then single tokens); after each step the blocks it completed
    must have their means in the coarser cache and no others.  Every position's row is then compared with the plain
    function.  One key just inside the window's far edge, one just outside it (in no block yet), the last token of the
    newest visible block and the first token of the next block carry marks that the query is aligned with, each in a
    row of its own: a window or a block count that is one off moves that row's output to another value."""
    from thintensor_b200.kernels import api

    # the steps that fill the cache; sequence 1 is one step behind so that the two complete different blocks in a step
    cuts = [1, 2, pool, max(1, pool - 1), 3 * pool + 1, window, 1, 1, 1]
    scale, total = 0.25, max(3 * max(window, pool) + 2 * pool + 7, sum(cuts) + pool + 3)
    cuts.append(total - sum(cuts))
    pools = Pools(2, total, kv_heads, dim, dim, act_dtype, 31)
    coarse = Pools(2, total // pool + 1, kv_heads, dim, dim, act_dtype, 32)
    keys = [randn(total, kv_heads, dim, seed=33 + b) for b in range(2)]
    values = [randn(total, kv_heads, dim, seed=35 + b) for b in range(2)]
    q = randn(2, total, heads, dim, seed=37)
    last = total - 1
    nb = plain.visible_blocks(last, window, pool)
    marks = {"inside": last - window + 1, "outside": last - window, "block_in": nb * pool - 1, "block_out": nb * pool}
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    done = [0, 0]
    for step, count in enumerate(cuts + [0]):
        news = [count if step < len(cuts) else 0, cuts[step - 1] if step > 0 else 0]
        live = [b for b in range(2) if news[b] > 0]
        before = [done[b] for b in live]
        for b in live:
            for p in range(done[b], done[b] + news[b]):
                pools.put(b, p, keys[b][p], values[b][p])
        table = pools.table[live].contiguous()
        mean_table = coarse.table[live].contiguous()
        new_live = [news[b] for b in live]
        api.pool_blocks(pools.k, pools.v, table, coarse.k, coarse.v, mean_table, cu_of(new_live), ints(before), len(live),
                        max(new_live) // pool + 1, kv_heads, dim, dim, pool, status)
        for b in live:
            done[b] += news[b]
        for b in range(2):
            for n in range(total // pool + 1):
                if n < done[b] // pool:
                    want = torch.stack([pools.key(b, p) for p in range(n * pool, n * pool + pool)]).mean(0)
                    assert float((coarse.key(b, n) - want).abs().max()) <= (1e-6 if act_dtype == torch.float32 else 2e-2), (step, b, n)
                    want = torch.stack([pools.value(b, p) for p in range(n * pool, n * pool + pool)]).mean(0)
                    assert float((coarse.value(b, n) - want).abs().max()) <= (1e-6 if act_dtype == torch.float32 else 2e-2), (step, b, n)
                else:
                    assert float(coarse.key(b, n)[0, 0]) == 50.0, (step, b, n)      # untouched
    assert done == [total, total]
    # rows: every position of sequence 0 as a prompt; the marked rows of sequence 1 as single decoded tokens
    kb = [torch.stack([pools.key(b, p) for p in range(total)]) for b in range(2)]
    vb = [torch.stack([pools.value(b, p) for p in range(total)]) for b in range(2)]
    km = [torch.stack([coarse.key(b, n) for n in range(total // pool)]) for b in range(2)]
    vm = [torch.stack([coarse.value(b, n) for n in range(total // pool)]) for b in range(2)]
    tol = 2e-5 if act_dtype == torch.float32 else 3e-2
    qd = q.to(act_dtype)
    out = torch.empty(total, heads * dim, dtype=act_dtype, device=DEV)
    for splits in (1, 3):
        part_acc = torch.empty(total * heads * splits * dim, dtype=torch.float32, device=DEV)
        part_ml = torch.empty(total * heads * splits * 2, dtype=torch.float32, device=DEV)
        api.pooled_window_attention(qd[0].reshape(total, -1).to(DEV), pools.k, pools.v, pools.table[:1].contiguous(), coarse.k, coarse.v,
                                    coarse.table[:1].contiguous(), pool, cu_of([total]), ints([0]), 1, total, heads, kv_heads, dim, scale, cap,
                                    window, splits, out, part_acc, part_ml, status)
        for i in range(total):
            for h in range(heads):
                want = plain_pooled_row(qd[0, i].double(), kb[0], vb[0], km[0], vm[0], i, h, heads // kv_heads, window, pool, scale, cap)
                assert float((out[i].double().cpu().view(heads, dim)[h] - want).abs().max()) <= tol, (splits, i, h)
    for name, position in marks.items():
        if not 0 <= position < total:
            continue
        # the query of the last position points at the marked token's key, strongly
        mark = randn(dim, seed=40, scale=2.0)
        pools.put(1, position, mark.expand(kv_heads, dim), values[1][position] + 9.0)
        kb1, vb1 = kb[1].clone(), vb[1].clone()
        kb1[position], vb1[position] = pools.key(1, position), pools.value(1, position)
        n = position // pool
        if n < total // pool:       # its block's means change with it
            for p_kv, means, rows in ((pools.k, km[1], kb1), (pools.v, vm[1], vb1)):
                means[n] = rows[n * pool: n * pool + pool].mean(0)
            coarse.put(1, n, km[1][n], vm[1][n])
            km[1][n], vm[1][n] = coarse.key(1, n), coarse.value(1, n)
        query = (mark * 3.0).expand(heads, dim).to(act_dtype)
        one = torch.empty(1, heads * dim, dtype=act_dtype, device=DEV)
        for splits in (1, 4):       # a decoding step, its keys whole and in slices
            part_acc = torch.empty(heads * splits * dim, dtype=torch.float32, device=DEV)
            part_ml = torch.empty(heads * splits * 2, dtype=torch.float32, device=DEV)
            one.fill_(7.0)
            api.pooled_window_attention(query.reshape(1, -1).to(DEV), pools.k, pools.v, pools.table[1:].contiguous(), coarse.k, coarse.v,
                                        coarse.table[1:].contiguous(), pool, cu_of([1]), ints([last]), 1, 1, heads, kv_heads, dim, scale, cap, window,
                                        splits, one, part_acc, part_ml, status)
            for h in range(heads):
                want = plain_pooled_row(query.double(), kb1, vb1, km[1], vm[1], last, h, heads // kv_heads, window, pool, scale, cap)
                # the marked value is large: bfloat16 rounds an output of that size by up to half a unit in its last place
                assert float((one[0].double().cpu().view(heads, dim)[h] - want).abs().max()) <= tol * max(1.0, float(want.abs().max())), (name, position, splits, h)
        kb[1], vb[1] = kb1, vb1
    assert int(status.item()) == 0
