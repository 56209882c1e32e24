"""The Sogidra decoder in the engine against the plain implementation, under every way of cutting the work: whole
prompts around the windows', the pooled blocks' and the cache blocks' edges; prompts cut into portions down to two
tokens; the last tokens and the very first tokens one by one; batches of unequal requests against each alone, with
slots, token blocks and blocks of means that are freed and used again; long decoding in which a window passes over
decoded tokens and the first token still counts; greedy generation through the runtime's own entry point; the trace
replay program and the command line as subprocesses; configurations drawn from a seed; and one-layer models whose
weights make a single far key, a window's edge or a block's edge decide the output."""
from __future__ import annotations

import pytest
import torch

from conftest import token_ids
from sogidra_models import CONFIGS, oracle_float32_drift, oracle_logits, oracle_sensitivity, write_model

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
NAMES = list(CONFIGS)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("sogidra")
    made = {}

    def get(name: str, dtype: str):
        stored = "float32" if dtype == "float32" else "bfloat16"
        if (name, stored) not in made:
            made[(name, stored)] = write_model(base / f"{name}-{stored}", name, stored)
        return made[(name, stored)]

    return get


def load(folder, dtype):
    import thintensor_b200

    return thintensor_b200.load_model(folder, dtype=dtype, device="cuda")


def most(name: str) -> int:
    return CONFIGS[name]["max_positions"]


class Judge:
    """Compares rows of logits with the plain implementation's.  float32: every logit within 5e-5 of the request's largest
    one, plus ten times what float32 rounding alone does to the plain implementation at that position (a differential
    layer that subtracts two nearly equal maps before its norm carries rounding far).  bfloat16: the cosine with the plain logits, position by position, against ``1 - cos <= 1e-3 + 4 s``, s being how
    far the plain implementation itself moves at that position when it narrows its activations to bfloat16 where an engine
    has to; over a test at most one position in fifty (and one) may exceed its bound, and the mean cosine must be at
    least 0.995.  A wrong key, a window that is one token off or a lost block moves most positions after it by far more."""

    def __init__(self, dtype, folder):
        self.dtype, self.folder, self.away, self.over, self.notes = dtype, folder, [], 0, []

    def add(self, got, tokens, rows, what):
        rows = list(rows)
        want = oracle_logits(self.folder, tokens)[rows]
        got = got.double().cpu().reshape(-1, got.shape[-1])
        assert got.shape == want.shape and torch.isfinite(got).all(), what
        if self.dtype == "float32":
            scale = max(1.0, float(want.abs().max()))
            err = (got - want).abs().max(dim=-1).values
            bound = 5e-5 * scale + 10.0 * oracle_float32_drift(self.folder, tokens)[rows]
            worst = int((err / bound).argmax())
            assert float(err[worst]) <= float(bound[worst]), f"{what}: position {rows[worst]}: max |diff| {float(err[worst]):.3e}, bound {float(bound[worst]):.3e}, logits up to {scale:.3f}"
            return
        away = 1.0 - torch.nn.functional.cosine_similarity(got, want, dim=-1)
        bound = 1e-3 + 4.0 * oracle_sensitivity(self.folder, tokens)[rows]
        bad = away > bound
        if bool(bad.any()):
            worst = int((away / bound).argmax())
            self.notes.append(f"{what}: position {rows[worst]} has cosine {1 - float(away[worst]):.5f}, rounding alone allows {1 - float(bound[worst]):.5f}")
        self.over += int(bad.sum())
        self.away.append(away)

    def done(self):
        if self.dtype == "bfloat16":
            away = torch.cat(self.away)
            assert self.over <= 1 + away.numel() // 50, f"{self.over} of {away.numel()} positions beyond their bound; " + "; ".join(self.notes[:4])
            assert float(1.0 - away.mean()) >= 0.995, f"mean cosine {float(1.0 - away.mean()):.5f}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_alone(folders, name, dtype):
    """Every position of prompts whose lengths lie around the windows' edges (1, 9, 21, 33, 100, 150), the ends of
    pooled blocks (5, 8, 16, 30, 64) and the cache's block borders (64, 128, 192)."""
    from thintensor_b200.engine.engine import Entry

    folder = folders(name, dtype)
    judge = Judge(dtype, folder)
    engine = load(folder, dtype).new_engine(max_tokens=512, max_sequences=2)
    for seed, length in enumerate([1, 2, 3, 5, 9, 10, 21, 22, 26, 33, 34, 41, 63, 64, 65, 100, 116, 129, 150, 151, 193, 214, 215, 290]):
        tokens = token_ids(CONFIGS[name]["vocab"], min(length, most(name)), 100 + seed)
        slot = engine.open()
        logits = engine.step([Entry(slot, tokens, list(range(len(tokens))))])
        engine.close(slot)
        engine.check_status()
        judge.add(logits, tokens, range(len(tokens)), f"{name} whole length {length}")
    assert engine.cache.free_blocks == engine.cache.num_blocks
    judge.done()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_in_portions(folders, name, dtype):
    """One prompt cut into steps of several sizes, down to two tokens and one: keys, the means of blocks that a cut
    divides, and the layers that read another layer's keys all continue across the cuts."""
    from thintensor_b200.engine.engine import Entry

    folder = folders(name, dtype)
    judge = Judge(dtype, folder)
    engine = load(folder, dtype).new_engine(max_tokens=512, max_sequences=2)
    tokens = token_ids(CONFIGS[name]["vocab"], 190, 210)
    for cuts in ([2, 2, 2, 1, 3, 11, 2, 41, 2, 64, 20, 40], [61, 3, 1, 1, 2, 82, 40], [16, 16, 32, 1, 85, 19, 21], [50, 140]):
        assert sum(cuts) == len(tokens)
        slot = engine.open()
        got, at = [], 0
        for count in cuts:
            got.append(engine.step([Entry(slot, tokens[at: at + count], list(range(count)))]))
            at += count
        engine.close(slot)
        engine.check_status()
        judge.add(torch.cat(got), tokens, range(len(tokens)), f"{name} portions {cuts}")
    judge.done()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_long_prompt_in_large_portions(folders, name, dtype):
    """Portions of about a hundred tokens far into a sequence, beside a second request in portions of another size: the
    window layers have by then given token blocks back, and a portion's first tokens see blocks of means and window
    tokens that earlier portions wrote."""
    from thintensor_b200.engine.engine import Entry

    folder = folders(name, dtype)
    judge = Judge(dtype, folder)
    engine = load(folder, dtype).new_engine(max_tokens=1024, max_sequences=2)
    sizes = (110, 90, 100) if most(name) < 400 else (150, 130, 120)
    tokens = token_ids(CONFIGS[name]["vocab"], sum(sizes), 215)
    other = token_ids(CONFIGS[name]["vocab"], 240, 216)
    a, b = engine.open(), engine.open()
    got, at = [], 0
    for step, count in enumerate(sizes):
        rows = [0, 1, count // 2, count - 2, count - 1]
        entries = [Entry(a, tokens[at: at + count], rows)]
        if step < 2:
            entries.append(Entry(b, other[120 * step: 120 * step + 120], [119]))
        out = engine.step(entries)
        got.append((at, rows, out))
        at += count
    engine.check_status()
    for at, rows, out in got:
        judge.add(out[: len(rows)], tokens, [at + r for r in rows], f"{name} portion at {at}")
    judge.add(torch.stack([out[len(rows)] for _, rows, out in got[:2]]), other, [119, 239], f"{name} the request beside it")
    judge.done()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_pieces_of_a_step(folders, name, dtype):
    """A step larger than the engine's limit runs in pieces; a sequence may straddle two of them."""
    from thintensor_b200.engine.engine import Entry

    folder = folders(name, dtype)
    judge = Judge(dtype, folder)
    engine = load(folder, dtype).new_engine(max_tokens=512, max_sequences=3, max_step_tokens=50)
    prompts = [token_ids(CONFIGS[name]["vocab"], n, 220 + n) for n in (70, 9, 45)]
    slots = [engine.open() for _ in prompts]
    logits = engine.step([Entry(s, p, [0, len(p) // 2, len(p) - 1]) for s, p in zip(slots, prompts)])
    engine.check_status()
    for i, p in enumerate(prompts):
        judge.add(logits[3 * i: 3 * i + 3], p, [0, len(p) // 2, len(p) - 1], f"{name} pieces, prompt {i}")
    judge.done()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_tokens_and_first_tokens_one_by_one(folders, name, dtype):
    """Decoding across the windows' edges (the prompt ends before them), across the ends of pooled blocks and across
    cache block borders, and from an empty slot."""
    from thintensor_b200.engine.engine import Entry

    folder = folders(name, dtype)
    judge = Judge(dtype, folder)
    engine = load(folder, dtype).new_engine(max_tokens=512, max_sequences=2)
    vocab = CONFIGS[name]["vocab"]
    for seed, (head, length) in enumerate([(4, 45), (61, 110), (120, 230)]):
        tokens = token_ids(vocab, length, 230 + seed)
        slot = engine.open()
        got = [engine.step([Entry(slot, tokens[:head], [head - 1])])]
        for t in range(head, length):
            got.append(engine.step([Entry(slot, [tokens[t]], [0])]))
        engine.close(slot)
        engine.check_status()
        judge.add(torch.cat(got), tokens, range(head - 1, length), f"{name} tail of length {length}")
    tokens = token_ids(vocab, 40, 240)                  # from an empty slot, token by token, past the short windows
    slot = engine.open()
    got = [engine.step([Entry(slot, [t], [0])]) for t in tokens]
    engine.close(slot)
    judge.add(torch.cat(got), tokens, range(len(tokens)), f"{name} first tokens")
    assert engine.cache.free_blocks == engine.cache.num_blocks
    judge.done()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_with_reuse(folders, name, dtype):
    """Batches of unequal prompts, each request then continued one token per step to its own length, so shorter requests
    leave earlier; the next batch gets the slots, token blocks and blocks of means that the last one gave back."""
    from thintensor_b200.engine.engine import Entry

    folder = folders(name, dtype)
    judge = Judge(dtype, folder)
    vocab = CONFIGS[name]["vocab"]
    batches = [
        [(5, 9), (9, 40), (1, 2), (17, 30)],
        [(70, 75), (1, 25), (40, 41)],
        [(64, 70), (3, 67), (128, 170), (20, 33)],
    ]
    room = max(sum(-(-total // 64) * 64 for _, total in batch) for batch in batches)
    engine = load(folder, dtype).new_engine(max_tokens=room, max_sequences=4)
    seed = 300
    for batch in batches:
        requests = []
        for prompt_len, total in batch:
            seed += 1
            requests.append({"tokens": token_ids(vocab, total, seed), "at": prompt_len, "total": total, "slot": engine.open(), "got": []})
        logits = engine.step([Entry(r["slot"], r["tokens"][: r["at"]], [r["at"] - 1]) for r in requests])
        for row, r in enumerate(requests):
            r["got"].append(logits[row])
        while True:
            for r in requests:
                if r["at"] >= r["total"] and r["slot"] is not None:
                    engine.close(r["slot"])
                    r["slot"] = None
            live = [r for r in requests if r["slot"] is not None]
            if not live:
                break
            logits = engine.step([Entry(r["slot"], [r["tokens"][r["at"]]], [0]) for r in live])
            for row, r in enumerate(live):
                r["got"].append(logits[row])
                r["at"] += 1
        engine.check_status()
        for r, (prompt_len, total) in zip(requests, batch):
            judge.add(torch.stack(r["got"]), r["tokens"], range(prompt_len - 1, total), f"{name} request {prompt_len}->{total} in a batch")
    assert engine.cache.free_blocks == engine.cache.num_blocks
    for group in engine.cache.kv_groups:
        assert group.table.pool.free_count == group.num_blocks
    judge.done()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_long_decoding(folders, name, dtype):
    """A prompt and then 170 decoded tokens (fewer where the model has fewer positions), most of them replayed from the
    engine's captured decode step: every window passes over decoded tokens and blocks of decoded tokens get their
    means.  The first token still shows in the plain implementation's last logits (through a differential layer's keys,
    or through the first block's mean)."""
    from thintensor_b200.engine.engine import Entry

    folder = folders(name, dtype)
    judge = Judge(dtype, folder)
    engine = load(folder, dtype).new_engine(max_tokens=512, max_sequences=2)
    vocab = CONFIGS[name]["vocab"]
    head, total = (120, 290) if most(name) < 400 else (180, 350)
    tokens = token_ids(vocab, total, 400)
    want = oracle_logits(folder, tokens)
    other = oracle_logits(folder, [(tokens[0] + 1) % vocab] + tokens[1:])
    assert float((want[-1] - other[-1]).abs().max()) > 1e-3 * float(want.abs().max())      # token 0 matters at the end
    slot = engine.open()
    got = [engine.step([Entry(slot, tokens[:head], [head - 1])])]
    for t in range(head, total):
        got.append(engine.step([Entry(slot, [tokens[t]], [0])]))
    engine.close(slot)
    engine.check_status()
    assert engine.graph_replays > 100
    judge.add(torch.cat(got), tokens, range(head - 1, total), f"{name} long decoding")
    judge.done()


@pytest.mark.parametrize("name", NAMES)
def test_logits_do_not_depend_on_the_batch(folders, name):
    """float32: a request's logits inside a batch equal those it gets alone up to the rounding of sums taken in another
    order, whatever else runs."""
    from thintensor_b200.engine.engine import Entry

    folder = folders(name, "float32")
    engine = load(folder, "float32").new_engine(max_tokens=1024, max_sequences=5, step_graphs=False)
    vocab = CONFIGS[name]["vocab"]
    prompts = [token_ids(vocab, n, 500 + n) for n in (33, 70, 17, 5)]
    alone = []
    for p in prompts:
        slot = engine.open()
        alone.append(engine.step([Entry(slot, p, [len(p) - 1])]))
        engine.close(slot)
    slots = [engine.open() for _ in prompts]
    together = engine.step([Entry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    alone = torch.cat(alone)
    # sums taken in another order round differently, and a differential layer carries that as far as it carries the
    # plain implementation's own rounding to float32 at that position
    carried = torch.stack([oracle_float32_drift(folder, p)[-1] for p in prompts]).to(alone.device)
    err = (together - alone).abs().max(dim=-1).values
    # up to 16 tokens alone go through the exact product's form for few rows, which sums k in another order than the
    # tiled form that the batch uses; longer requests use the tiled form both times
    few = torch.tensor([16.0 if len(p) <= 16 else 4.0 for p in prompts], device=alone.device)
    assert bool((err <= 2e-6 * float(alone.abs().max()) + few * carried).all()), (err, carried)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation(folders, name, dtype):
    """``Runtime.generate`` (scheduler, decode graph, sampler) against greedy decoding with the plain implementation.
    A step whose two best logits are nearly tied is allowed to differ; what follows it is then not compared."""
    folder = folders(name, dtype)
    runtime = load(folder, dtype)
    vocab = CONFIGS[name]["vocab"]
    prompts = [token_ids(vocab, n, 600 + n) for n in (7, 30, 66, 3, 18)]
    new = runtime.generate(prompts, max_new_tokens=10, stop_ids=(), batch_size=3)
    for prompt, got in zip(prompts, new):
        assert len(got) == 10
        sequence = list(prompt)
        for token in got:
            logits = oracle_logits(folder, sequence)[-1]
            best = torch.topk(logits, 2)
            if int(best.indices[0]) != token:
                margin = float(best.values[0] - logits[token])
                if dtype == "bfloat16" and float(oracle_sensitivity(folder, sequence)[-1]) > 1e-3:
                    break
                assert margin < (1e-3 if dtype == "float32" else 0.5), f"{name}: generated {token}, the plain model says {int(best.indices[0])} by {margin}"
                break
            sequence.append(token)


def test_generation_stops_at_the_last_position(folders):
    """A model has as many position vectors as its table has rows: a step that would pass them is refused."""
    from thintensor_b200.engine.engine import Entry, StepError

    folder = folders("c", "float32")
    engine = load(folder, "float32").new_engine(max_tokens=512, max_sequences=1)
    slot = engine.open()
    engine.step([Entry(slot, token_ids(CONFIGS["c"]["vocab"], most("c"), 1), [most("c") - 1])])
    with pytest.raises(StepError):
        engine.step([Entry(slot, [1], [0])])


def test_what_the_cache_holds(folders):
    """A window layer keeps the last max(window, block) tokens and, in a second group, one entry per block; a layer that
    reads another layer's keys has no storage of its own; a differential layer keeps rows of two maps."""
    engine = load(folders("a", "float32"), "float32").new_engine(max_tokens=256, max_sequences=2)
    needs = sorted((g.need.kv_heads, g.need.head_dim, g.need.v_dim, g.need.window or 0, g.need.every, len(g.runs)) for g in engine.cache.kv_groups)
    assert needs == [(1, 40, 40, 0, 5, 1), (1, 40, 40, 21, 1, 1), (2, 48, 40, 0, 1, 1)]
    assert len(engine.cache.state_groups) == 0
    engine = load(folders("b", "float32"), "float32").new_engine(max_tokens=256, max_sequences=2)
    windows = sorted((g.need.window or 0, g.need.every) for g in engine.cache.kv_groups)
    assert windows == [(0, 1), (0, 30), (0, 64), (1, 1), (30, 1), (150, 1)]
