"""The Kerepel decoder in the engine against the plain implementation, under every way of cutting the work: whole
prompts around the windows' and the cache blocks' edges; prompts cut into portions down to two tokens and one; the last
tokens and the very first tokens one by one; batches of unequal requests against each alone, with slots, blocks and
states (convolution tails, previous tokens) that are freed and used again; long decoding past windows and block borders,
replayed from CUDA graphs; a marked far token that only the unwindowed layers can carry; greedy generation through the
runtime's own entry point; the trace replay program and the command line as subprocesses; configurations drawn from a seed."""
from __future__ import annotations

import pytest
import torch

from conftest import token_ids
from kerepel_models import CONFIGS, Judge, oracle_logits, oracle_sensitivity, write_model

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
NAMES = list(CONFIGS)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("kerepel")
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


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_alone(folders, name, dtype):
    """Lengths around the windows' edges (21, 40, 70, 100, 150), the convolutions' taps and the cache's block borders."""
    from thintensor_b200.engine.engine import Entry

    folder = folders(name, dtype)
    judge = Judge(dtype, folder)
    engine = load(folder, dtype).new_engine(max_tokens=512, max_sequences=2)
    for seed, length in enumerate([1, 2, 3, 4, 5, 20, 21, 22, 40, 41, 63, 64, 65, 70, 71, 100, 101, 129, 150, 151, 230]):
        tokens = token_ids(CONFIGS[name]["vocab"], length, 100 + seed)
        slot = engine.open()
        logits = engine.step([Entry(slot, tokens, list(range(length)))])
        engine.close(slot)
        engine.check_status()
        judge.add(logits, tokens, range(length), f"{name} whole length {length}")
    assert engine.cache.free_blocks == engine.cache.num_blocks
    judge.done()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_in_portions(folders, name, dtype):
    """One prompt cut into steps of several sizes, down to two tokens and one: keys, latents, the convolutions' tails (a
    portion shorter than the taps leaves part of the old tail in place) and the previous token all continue across the cuts."""
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
    """Portions of more than a hundred tokens far into a sequence, beside a second request: a window has by then given
    blocks back, and a portion's first tokens look back into blocks that earlier portions wrote."""
    from thintensor_b200.engine.engine import Entry

    folder = folders(name, dtype)
    judge = Judge(dtype, folder)
    engine = load(folder, dtype).new_engine(max_tokens=1024, max_sequences=2)
    tokens = token_ids(CONFIGS[name]["vocab"], 420, 215)
    other = token_ids(CONFIGS[name]["vocab"], 300, 216)
    a, b = engine.open(), engine.open()
    got, at = [], 0
    for step, count in enumerate((150, 130, 140)):
        rows = [0, 1, 2, count // 2, count - 2, count - 1]
        entries = [Entry(a, tokens[at: at + count], rows)]
        if step < 2:
            entries.append(Entry(b, other[150 * step: 150 * step + 150], [149]))
        out = engine.step(entries)
        got.append((at, rows, out))
        at += count
    engine.check_status()
    for at, rows, out in got:
        judge.add(out[: len(rows)], tokens, [at + r for r in rows], f"{name} portion at {at}")
    judge.add(torch.stack([out[len(rows)] for _, rows, out in got[:2]]), other, [149, 299], f"{name} the request beside it")
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
    """Prefill against token-by-token decoding: across a window's edge (the prompt ends before it), across block borders,
    and from an empty slot (the convolutions start from zeros, the pair table from its last row)."""
    from thintensor_b200.engine.engine import Entry

    folder = folders(name, dtype)
    judge = Judge(dtype, folder)
    engine = load(folder, dtype).new_engine(max_tokens=512, max_sequences=2)
    vocab = CONFIGS[name]["vocab"]
    for seed, (head, length) in enumerate([(4, 45), (61, 110), (120, 170)]):
        tokens = token_ids(vocab, length, 230 + seed)
        slot = engine.open()
        got = [engine.step([Entry(slot, tokens[:head], [head - 1])])]
        for t in range(head, length):
            got.append(engine.step([Entry(slot, [tokens[t]], [0])]))
        engine.close(slot)
        engine.check_status()
        judge.add(torch.cat(got), tokens, range(head - 1, length), f"{name} tail of length {length}")
    tokens = token_ids(vocab, 30, 240)
    slot = engine.open()
    got = [engine.step([Entry(slot, [t], [0])]) for t in tokens]
    engine.close(slot)
    judge.add(torch.cat(got), tokens, range(len(tokens)), f"{name} first tokens")
    judge.done()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_with_reuse(folders, name, dtype):
    """Batches of unequal prompts, each request then continued one token per step to its own length, so shorter requests
    leave earlier; the next batch gets the slots, blocks and states that the last one gave back."""
    from thintensor_b200.engine.engine import Entry

    folder = folders(name, dtype)
    judge = Judge(dtype, folder)
    vocab = CONFIGS[name]["vocab"]
    batches = [
        [(5, 9), (9, 40), (1, 2), (17, 30)],
        [(70, 75), (1, 25), (40, 41)],
        [(64, 70), (3, 67), (128, 160), (20, 33)],
    ]
    most = max(sum(-(-total // 64) * 64 for _, total in batch) for batch in batches)
    engine = load(folder, dtype).new_engine(max_tokens=most, max_sequences=4)
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
    judge.done()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_long_decoding(folders, name, dtype):
    """A long prompt and 150 decoded tokens, most of them replayed from the engine's captured decode step; the windowed
    groups give blocks back on the way and every window's edge passes over decoded tokens.  The first token still shows
    at the end: only the unwindowed latent layers can carry it that far."""
    from thintensor_b200.engine.engine import Entry

    folder = folders(name, dtype)
    judge = Judge(dtype, folder)
    engine = load(folder, dtype).new_engine(max_tokens=512, max_sequences=2)
    vocab = CONFIGS[name]["vocab"]
    tokens = token_ids(vocab, 330, 400)
    want = oracle_logits(folder, tokens)
    other = oracle_logits(folder, [(tokens[0] + 1) % vocab] + tokens[1:])
    assert float((want[-1] - other[-1]).abs().max()) > 1e-4 * float(want.abs().max())      # token 0 matters at the end
    slot = engine.open()
    got = [engine.step([Entry(slot, tokens[:180], [179])])]
    for t in range(180, 330):
        got.append(engine.step([Entry(slot, [tokens[t]], [0])]))
    engine.close(slot)
    engine.check_status()
    assert engine.graph_replays > 100
    judge.add(torch.cat(got), tokens, range(179, 330), f"{name} long decoding")
    judge.done()


@pytest.mark.parametrize("name", NAMES)
def test_logits_do_not_depend_on_the_batch(folders, name):
    """float32: a request's logits inside a batch equal those it gets alone up to the rounding of sums taken in another
    order, whatever else runs."""
    from thintensor_b200.engine.engine import Entry

    folder = folders(name, "float32")
    engine = load(folder, "float32").new_engine(max_tokens=1024, max_sequences=4, step_graphs=False)
    vocab = CONFIGS[name]["vocab"]
    prompts = [token_ids(vocab, n, 500 + n) for n in (33, 70, 5)]
    alone = []
    for p in prompts:
        slot = engine.open()
        alone.append(engine.step([Entry(slot, p, [len(p) - 1])]))
        engine.close(slot)
    slots = [engine.open() for _ in prompts]
    together = engine.step([Entry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    alone = torch.cat(alone)
    assert float((together - alone).abs().max()) <= 2e-6 * float(alone.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation(folders, name, dtype):
    """``Runtime.generate`` (scheduler, decode graph, sampler) against greedy decoding with the plain implementation.
    A step whose two best logits are nearly tied is allowed to differ, and in bfloat16 so is one at a position that the
    rounding of activations alone moves far (a router's close call); what follows it is then not compared."""
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
                near = 1e-3 if dtype == "float32" else 0.15 * float(logits.std())        # bfloat16: a small share of the logits' spread
                assert margin < near, f"{name}: generated {token}, the plain model says {int(best.indices[0])} by {margin}"
                break
            sequence.append(token)


def test_what_the_cache_holds(folders):
    """A reader keeps no keys of its own and its source's group keeps what the wider of the two windows sees; latent
    attention keeps one row per token and no value pool; convolutions have their tails as states, readers only the queries'."""
    runtime = load(folders("a", "float32"), "float32")
    assert runtime.model.device_driven
    engine = runtime.new_engine(max_tokens=128, max_sequences=2)
    needs = sorted((g.need.kv_heads, g.need.head_dim, g.need.v_dim, g.need.window, len(g.runs)) for g in engine.cache.kv_groups)
    assert needs == [(1, 48, 0, None, 1), (3, 16, 24, 40, 1)]
    shapes = sorted((tuple(g.need.shape), g.need.dtype, len(g.runs)) for g in engine.cache.state_groups)
    assert shapes == sorted([((), torch.int32, 1), ((3, 3 * 16 + 3 * 16 + 3 * 24), torch.float32, 1), ((1, 3 * 16), torch.float32, 1)])
    engine = load(folders("b", "float32"), "float32").new_engine(max_tokens=128, max_sequences=2)
    needs = sorted((g.need.kv_heads, g.need.head_dim, g.need.v_dim, g.need.window, len(g.runs)) for g in engine.cache.kv_groups)
    assert needs == [(1, 32, 32, 150, 1), (1, 40, 0, None, 1)]


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("c", "bfloat16"), ("b", "bfloat16")])
def test_trace_replay_as_a_subprocess(folders, tmp_path, name, dtype):
    """``bin/trace_run`` chooses the model class by config.json: prompts of unequal lengths start together, go on one
    token each, the shorter ones end earlier, and a second batch reuses what the first gave back."""
    from test_trace_run_gpu import read_step, run_trace

    folder = folders(name, dtype)
    vocab = CONFIGS[name]["vocab"]
    requests = {f"q{i}": token_ids(vocab, n, 700 + i) for i, n in enumerate([40, 9, 75, 66])}
    prompt_len = {"q0": 7, "q1": 1, "q2": 64, "q3": 60}
    judge = Judge(dtype, folder)
    steps, expect, n = [], [], 0
    for batch in (["q0", "q2", "q1"], ["q3"]):
        at = {k: prompt_len[k] for k in batch}
        steps.append({"step": n, "entries": [{"id": k, "tokens": requests[k][: at[k]], "want": [0, at[k] - 1]} for k in batch], "end": []})
        expect.append((n, [(k, place) for k in batch for place in (0, at[k] - 1)]))
        n += 1
        live = list(batch)
        while live:
            entries, wanted, ending = [], [], []
            for k in live:
                entries.append({"id": k, "tokens": [requests[k][at[k]]], "want": [0] if at[k] % 2 else []})
                if at[k] % 2:
                    wanted.append((k, at[k]))
                at[k] += 1
                if at[k] == len(requests[k]):
                    ending.append(k)
            steps.append({"step": n, "entries": entries, "end": ending})
            expect.append((n, wanted))
            n += 1
            live = [k for k in live if k not in ending]
    run_trace(folder, dtype, tmp_path / "out", 192, steps)
    for step, wanted in expect:
        if not wanted:
            assert not (tmp_path / "out" / f"{step}.f32").exists()
            continue
        got = read_step(tmp_path / "out", step, vocab)
        for row, (k, place) in enumerate(wanted):
            judge.add(got[row: row + 1], requests[k], [place], f"{name} step {step} request {k}")
    judge.done()


def test_command_line(tmp_path):
    """``random`` writes a model folder from a config.json, ``run`` generates from it greedily, ``bench`` times it."""
    import json

    import plain_kerepel
    from test_cli_gpu import cli

    (tmp_path / "config.json").write_text(json.dumps(CONFIGS["a"]))
    folder = tmp_path / "model"
    assert cli("random", str(folder), "--config", str(tmp_path / "config.json"), "--seed", "5", "--dtype", "float32").strip() == str(folder)
    out = json.loads(cli("run", str(folder), "--prompt-token-ids", "5,17,3,100,42", "--max-new-tokens", "5", "--dtype", "fp32",
                         "--ignore-eos", "--json"))
    cfg, weights = plain_kerepel.read_model(folder)
    sequence = [5, 17, 3, 100, 42]
    for _ in range(5):
        sequence.append(int(plain_kerepel.forward(cfg, weights, sequence)[-1].argmax()))
    assert out["generated_token_ids"] == [sequence[5:]]
    bench = json.loads(cli("bench", str(folder), "--steps", "8", "--warmup", "3", "--prompt-len", "20", "--batch", "2", "--json"))
    assert bench["tokens_per_s"] > 0 and bench["prefill_tokens_per_s"] > 0


def random_config(seed: int) -> dict:
    """A configuration drawn from a seed: layer order, every size and every constant (sizes need not be multiples of
    anything: widths that are no multiple of 8 run the exact product in bfloat16 too)."""
    import random

    r = random.Random(seed)

    def latent():
        rot_dim = r.choice([2, 4, 8, 16, 40])
        mixer = {"heads": r.choice([1, 2, 4, 7]), "dim": r.choice([8, 20, 32, 72]), "rot_dim": rot_dim, "vdim": r.choice([6, 16, 34, 64]),
                 "kv_rank": r.choice([8, 24, 56, 136]), "scale": r.choice([0.1, 0.3, 0.05])}
        if r.random() < 0.85:
            mixer["rot"] = {"dims": rot_dim, "base": r.choice([100.0, 30000.0, 1e6])}
            if r.random() < 0.7:
                mixer["rot"]["scaling"] = {"factor": r.choice([1.0, 2.0, 8.0, 40.0]), "original": r.choice([16, 64, 4096]),
                                           "fast": r.choice([4.0, 32.0]), "slow": r.choice([0.5, 1.0, 2.0])}
        return mixer

    def attention(sources):
        if sources and r.random() < 0.5:
            index, source = r.choice(sources)
            mixer = {"heads": source["heads"], "kv_heads": source["kv_heads"], "dim": source["dim"], "vdim": source["vdim"], "kv_from": index}
        else:
            kv_heads = r.choice([1, 2, 3])
            mixer = {"heads": kv_heads * r.choice([1, 2, 4]), "kv_heads": kv_heads, "dim": r.choice([8, 16, 20, 48, 64]), "vdim": r.choice([8, 16, 36, 64])}
        mixer["scale"] = r.choice([0.1, 0.2, 0.35])
        if r.random() < 0.85:
            mixer["conv"] = r.choice([1, 2, 3, 4, 6])
        if r.random() < 0.85:
            mixer["mask"] = {"size": r.choice([1, 2, 7, 33, 64, 65, 100, 129])}
        if r.random() < 0.8:
            mixer["softcap"] = r.choice([5.0, 30.0, 50.0])
        return mixer

    def mlp():
        pick = r.random()
        if pick < 0.15:
            return None
        if pick < 0.45:
            return {"kind": "dense", "ff": r.choice([24, 50, 99, 160])}
        groups = r.choice([1, 2, 3, 4])
        size = r.choice([1, 2, 3])
        keep = r.randint(1, groups)
        out = {"kind": "moe", "expert": {"ff": r.choice([8, 24, 50]), "limit": r.choice([0.5, 1.0, 7.0])},
               "router": {"experts": groups * size, "top": r.randint(1, keep * size), "groups": {"count": groups, "keep": keep}}}
        if r.random() < 0.7:
            out["shared"] = {"ff": r.choice([8, 40, 72]), "limit": r.choice([0.75, 2.0])}
        return out

    layers, sources = [], []
    for index in range(r.choice([2, 3, 4, 5])):
        if r.random() < 0.4:
            layers.append({"type": "latent_attention", "mixer": latent(), "mlp": mlp()})
        else:
            mixer = attention(sources)
            if "kv_from" not in mixer:
                sources.append((index, mixer))
            layers.append({"type": "attention", "mixer": mixer, "mlp": mlp()})
    config = {"architecture": "Kerepel", "vocab": r.choice([50, 129, 300]), "width": r.choice([40, 90, 100, 128]),
              "norm": {"eps": r.choice([1e-6, 1e-5])}, "layers": layers}
    if r.random() < 0.8:
        config["logit_scale"] = r.choice([0.25, 0.7, 3.0])
    if r.random() < 0.8:
        config["token_side"] = {"dim": r.choice([1, 4, 8, 24])}
    if r.random() < 0.8:
        config["embedding"] = {"bigram": {"buckets": r.choice([1, 13, 257]), "mul_prev": r.choice([0, 1, 29, 1000003]), "mul_cur": r.choice([1, 19, 99991])}}
    return config


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16, 17, 18])
def test_configurations_drawn_from_a_seed(tmp_path, seed, dtype):
    """Whole, then a prompt and decoding beside a second request in the same batch, on models whose order of layers,
    sizes and constants are drawn at random."""
    from thintensor_b200.engine.engine import Entry

    config = random_config(seed)
    folder = write_model(tmp_path / f"seed{seed}", "", "float32" if dtype == "float32" else "bfloat16", config=config, seed=seed)
    vocab = config["vocab"]
    engine = load(folder, dtype).new_engine(max_tokens=512, max_sequences=3)
    judge = Judge(dtype, folder)
    first, second = token_ids(vocab, 150, 800 + seed), token_ids(vocab, 70, 900 + seed)
    slot = engine.open()
    judge.add(engine.step([Entry(slot, first, list(range(150)))]), first, range(150), f"seed {seed} whole")
    engine.close(slot)
    a, b = engine.open(), engine.open()
    got_a = [engine.step([Entry(a, first[:61], [60]), Entry(b, second[:3], [])])[0:1]]
    got_b = []
    for t in range(61, 150):
        entries = [Entry(a, [first[t]], [0])]
        if 3 + t - 61 < 70:
            entries.append(Entry(b, [second[3 + t - 61]], [0]))
        out = engine.step(entries)
        got_a.append(out[0:1])
        if len(entries) > 1:
            got_b.append(out[1:2])
    engine.check_status()
    judge.add(torch.cat(got_a), first, range(60, 150), f"seed {seed} first request")
    judge.add(torch.cat(got_b), second, range(3, 3 + len(got_b)), f"seed {seed} second request")
    judge.done()
