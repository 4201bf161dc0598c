"""The Relilix decoder in the engine against the plain implementation (plain_relilix.py): every mechanism in a model of
its own, whole prompts, prompts against token-by-token decoding, portions down to two tokens, unequal batches against
each request alone, slots, pages and rings that are used again, decoding across page borders and past every window, the
first tokens, other sizes (one head, one expert per token, heads that need padding, layers without taps, window, cap,
rotation or feed-forward), windows of hundreds of tokens, recorded steps, and greedy generation through the library's
own entry point."""
import pytest
import torch

import plain_relilix as plain
import tiny_relilix as tiny

pytestmark = pytest.mark.gpu

TOL_F32 = 3e-5            # largest |engine - plain| relative to the largest |logit| of the row: float32 sums against float64
# bfloat16: a row's error relative to the row's largest logit.  The yardstick is the plain implementation with roundings
# to bfloat16 where an engine stores activations: its distance from the exact result is what the storage format alone
# costs on this input.  The engine's typical row must be as close as the yardstick's (twice its median) and few rows
# may lie far beyond the yardstick's 90th percentile.  Both plain results use the experts that the engine itself chose
# (`RouterSpy`): a close call of a router that rounding turns is no error of the arithmetic, and behind a window of a few
# tokens one turned choice would colour every row that still sees the token.  The bfloat16 engines of these checks
# therefore run without recorded steps (a replayed recording calls no Python that could be watched); recorded bfloat16
# steps are compared with the unrecorded ones instead, and the float32 engine records as usual.
BF16_FACTOR, BF16_SLACK, BF16_ROWS_OVER = 2.0, 0.004, 0.1


class RouterSpy:
    """Records the experts that every routed feed-forward chooses: `steps[s][j]` is an int64 [rows, top] tensor for the
    j-th routed layer (in layer order) of the s-th step while the spy is active."""

    def __init__(self):
        self.steps = []

    def __enter__(self):
        from catena_models_b200 import kernels

        self._kernels, self._original = kernels, kernels.moe_route
        spy = self

        def route(ids, wts, perm, dest, work, h, w_router, tok_seq, top, *a, **k):
            out = spy._original(ids, wts, perm, dest, work, h, w_router, tok_seq, top, *a, **k)
            if not torch.cuda.is_current_stream_capturing():         # a step that is being recorded runs nothing yet
                spy.steps[-1].append(ids.view(-1, top).long().cpu())
            return out

        kernels.moe_route = route
        return self

    def __exit__(self, *exc):
        self._kernels.moe_route = self._original

    def begin_step(self):
        self.steps.append([])


def routed_layers(cfg):
    return [i for i, layer in enumerate(cfg["layers"]) if layer.get("mlp") and layer["mlp"]["kind"] == "moe"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("relilix")
    return {name: tiny.make_folder(tmp, name, seed=70 + i) for i, name in enumerate(tiny.ALL)}


@pytest.fixture(scope="module")
def plains(folders):
    return {name: tiny.load_plain(f) for name, f in folders.items()}


_models = {}


def model_for(folders, name, dtype, **kw):
    from catena_models_b200.api import Model

    if dtype == "bfloat16":
        kw.setdefault("use_graphs", False)
    key = (name, dtype, tuple(sorted(kw.items())))
    if key not in _models:
        _models[key] = Model.load(folders[name], dtype=dtype, max_tokens=8192, **kw)
    return _models[key]


def row_errs(got, ref):
    ref = ref.to(torch.float64).cpu()
    return (got.to(torch.float64).cpu() - ref).abs().amax(-1) / ref.abs().amax(-1)


def check(got, ref, dtype):
    """ref: the exact logits, or (exact, the yardstick's) for bfloat16."""
    same = None
    if isinstance(ref, tuple):
        ref, same = ref
    assert got.shape == ref.shape
    assert bool(torch.isfinite(got).all())
    errs = row_errs(got, ref)
    if dtype == "float32":
        assert float(errs.max()) < TOL_F32, float(errs.max())
    else:
        yard = row_errs(same, ref)
        assert float(errs.median()) < BF16_FACTOR * float(yard.median()) + BF16_SLACK, (float(errs.median()), float(yard.median()))
        far = 3.0 * float(torch.quantile(yard, 0.9)) + 4 * BF16_SLACK
        assert float((errs > far).double().mean()) <= BF16_ROWS_OVER, (errs, far)


_exact = {}


def exact(plains, name, tokens, dtype="float32", ids=None):
    """The plain logits; for bfloat16 (exact, yardstick), both with the experts `ids` ({layer: [T, top]})."""
    cfg, tensors = plains[name]
    if dtype == "bfloat16":
        if ids is None and routed_layers(cfg):
            raise ValueError("bfloat16 checks of a routed model follow the engine's own choice of experts")
        return (plain.forward(tokens, tensors, cfg, expert_ids=ids)[0],
                plain.forward(tokens, tensors, cfg, rd=plain.to_bf16, expert_ids=ids)[0])
    key = (name, tuple(tokens))
    if key not in _exact:
        _exact[key] = plain.forward(tokens, tensors, cfg)[0]
    return _exact[key]


def run_alone(engine, tokens, cuts, cfg=None):
    """One request through the engine in steps of the given sizes (the rest token by token); every logit.  With `cfg`:
    (logits, {layer: the experts the engine chose, [T, top]})."""
    (slot,) = engine.admit(1)
    out, at = [], 0
    with RouterSpy() as spy:
        try:
            for n in list(cuts) + [1] * len(tokens):
                if at >= len(tokens):
                    break
                part = tokens[at:at + n]
                spy.begin_step()
                out.append(engine.step([slot], [part], [list(range(len(part)))]).float().cpu())
                at += len(part)
            engine.check_errors()
        finally:
            engine.release([slot])
    if cfg is None:
        return torch.cat(out)
    layers = routed_layers(cfg)
    if any(len(step) != len(layers) for step in spy.steps):
        return torch.cat(out), None                       # recorded steps: nothing was seen
    return torch.cat(out), {layer: torch.cat([step[j] for step in spy.steps]) for j, layer in enumerate(layers)}


def alone_against_plain(engine, plains, name, tokens, cuts, dtype):
    got, ids = run_alone(engine, tokens, cuts, plains[name][0])
    check(got, exact(plains, name, tokens, dtype, ids if dtype == "bfloat16" else None), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", [n for n in tiny.ALL if n != "L"])
def test_whole_prompt(folders, plains, name, dtype):
    engine = model_for(folders, name, dtype).engine
    tokens = tiny.prompt(150, tiny.ALL[name]["vocab"], 1)
    alone_against_plain(engine, plains, name, tokens, [len(tokens)], dtype)


def test_streams_after_every_layer(folders, plains):
    """The float32 residual stream after every layer of a whole prompt, against the plain statement's."""
    from catena_models_b200.parts.parallel import PreNormBlock

    engine = model_for(folders, "A", "float32").engine
    cfg, tensors = plains["A"]
    tokens = tiny.prompt(90, cfg["vocab"], 5)
    want = []
    plain.forward(tokens, tensors, cfg, streams=want)
    got, original = [], PreNormBlock.forward

    def spy(self, rt, batch, h, n, state, next_norm):
        out = original(self, rt, batch, h, n, state, next_norm)
        got.append(out[0][:len(tokens)].detach().double().cpu())
        return out

    PreNormBlock.forward = spy
    try:
        run_alone(engine, tokens, [len(tokens)])
    finally:
        PreNormBlock.forward = original
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert float((g - w).abs().max() / w.abs().max()) < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "M", "attention", "latent", "moe"])
def test_prompt_then_token_by_token(folders, plains, name, dtype):
    """A prompt in one step, then tokens one by one (recorded decode steps from the second on): across page borders (64,
    128), past every window and every ring's end, and from the very first token on."""
    engine = model_for(folders, name, dtype).engine
    tokens = tiny.prompt(200, tiny.ALL[name]["vocab"], 2)
    alone_against_plain(engine, plains, name, tokens, [50], dtype)
    alone_against_plain(engine, plains, name, tokens, [1], dtype)


@pytest.mark.parametrize("name", ["A", "B", "C", "M"])
def test_portions_of_several_sizes(folders, plains, name):
    engine = model_for(folders, name, "float32").engine
    tokens = tiny.prompt(200, tiny.ALL[name]["vocab"], 3)
    ref = exact(plains, name, tokens)
    for cuts in ([2] * 100, [3, 61, 1, 64, 2, 69], [64, 64, 64, 8], [127, 2, 2, 69], [1, 1, 2, 5, 7, 100, 84]):
        check(run_alone(engine, tokens, cuts), ref, "float32")
    bf = model_for(folders, name, "bfloat16").engine
    alone_against_plain(bf, plains, name, tokens, [33, 2, 65, 100], "bfloat16")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "M"])
def test_unequal_batch_against_each_alone(folders, plains, name, dtype):
    """Four requests of unequal length start together and are decoded together; the shorter ones end earlier and
    their slots, pages and rings are taken by new requests while the others go on."""
    engine = model_for(folders, name, dtype).engine
    cfg = plains[name][0]
    vocab, layers = cfg["vocab"], routed_layers(cfg)
    lens, extra = [1, 70, 23, 131], [3, 9, 30, 12]
    toks = [tiny.prompt(n + e, vocab, 10 + i) for i, (n, e) in enumerate(zip(lens, extra))]
    slots = engine.admit(4)
    got = [[] for _ in toks]
    chosen = [{layer: [] for layer in layers} for _ in toks]          # per request and routed layer: the engine's experts

    def seen(step, owners):
        """Hand a step's recorded choices to the requests that own its rows (owners: (request, rows) in row order)."""
        if len(step) != len(layers):
            return
        for j, layer in enumerate(layers):
            at = 0
            for i, n in owners:
                if i is not None:
                    chosen[i][layer].append(step[j][at:at + n])
                at += n

    with RouterSpy() as spy:
        spy.begin_step()
        logits = engine.step(slots, [t[:n] for t, n in zip(toks, lens)], [list(range(n)) for n in lens]).float().cpu()
        seen(spy.steps[-1], list(enumerate(lens)))
        at = 0
        for i, n in enumerate(lens):
            got[i].append(logits[at:at + n])
            at += n
        live, pos = list(range(4)), list(lens)
        late = None
        while live:
            spy.begin_step()
            logits = engine.step([slots[i] for i in live], [[toks[i][pos[i]]] for i in live]).float().cpu()
            seen(spy.steps[-1], [(i, 1) for i in live])
            for r, i in enumerate(live):
                got[i].append(logits[r:r + 1])
                pos[i] += 1
            done = [i for i in live if pos[i] == len(toks[i])]
            for i in done:
                engine.release([slots[i]])
            live = [i for i in live if i not in done]
            if done and late is None and live:
                # a new request takes a slot that was just given back, while the others decode on
                late_tokens = tiny.prompt(40, vocab, 99)
                (s,) = engine.admit(1)
                assert s in [slots[i] for i in done]
                spy.begin_step()
                late = engine.step([s], [late_tokens], [list(range(40))]).float().cpu()
                late_ids = {layer: spy.steps[-1][j] for j, layer in enumerate(layers)} if len(spy.steps[-1]) == len(layers) else None
                engine.release([s])
    engine.check_errors()
    for i in range(4):
        ids = {layer: torch.cat(chosen[i][layer]) for layer in layers} if dtype == "bfloat16" else None
        check(torch.cat(got[i]), exact(plains, name, toks[i], dtype, ids), dtype)
    check(late, exact(plains, name, late_tokens, dtype, late_ids if dtype == "bfloat16" else None), dtype)


def test_mixed_step_of_started_and_new_requests(folders, plains):
    """One step in which a started request brings several tokens, another one token and a third its whole prompt."""
    engine = model_for(folders, "A", "float32").engine
    vocab = tiny.ALL["A"]["vocab"]
    a, b, c = tiny.prompt(90, vocab, 31), tiny.prompt(70, vocab, 32), tiny.prompt(66, vocab, 33)
    sa, sb, sc = engine.admit(3)
    engine.step([sa, sb], [a[:60], b[:69]], [[], []])
    logits = engine.step([sa, sb, sc], [a[60:], b[69:], c], [list(range(30)), [0], list(range(66))]).float().cpu()
    engine.check_errors()
    engine.release([sa, sb, sc])
    check(logits[:30], exact(plains, "A", a)[60:], "float32")
    check(logits[30:31], exact(plains, "A", b)[69:], "float32")
    check(logits[31:], exact(plains, "A", c), "float32")


@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding(folders, plains, name):
    """Hundreds of single tokens: every ring turns over several times, the growing caches cross several pages."""
    engine = model_for(folders, name, "float32").engine
    tokens = tiny.prompt(400, tiny.ALL[name]["vocab"], 4)
    check(run_alone(engine, tokens, [5]), exact(plains, name, tokens), "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windows_of_hundreds_of_tokens(folders, plains, dtype):
    """A window of 800 and no window over prompts of 1,000 tokens (the long-prompt attention kernels of the bfloat16
    engine), then single tokens that move the window on, and a portion on top of held tokens."""
    engine = model_for(folders, "L", dtype).engine
    tokens = tiny.prompt(1000, tiny.ALL["L"]["vocab"], 6)
    ref = exact(plains, "L", tokens, dtype)
    check(run_alone(engine, tokens, [960]), ref, dtype)
    check(run_alone(engine, tokens, [700, 300]), ref, dtype)


@pytest.mark.parametrize("name", ["A", "M"])
def test_recorded_prompt_classes(folders, plains, name):
    """Prompts of one class of shapes (rows rounded up to 64, the same number of wanted places) run as a replayed
    recording from the third on, with rows of padding behind the tokens; so do portions on top of held tokens."""
    engine = model_for(folders, name, "float32").engine
    vocab = tiny.ALL[name]["vocab"]
    before = len(engine._prompt_graphs)
    got, ref = [], []
    for n in (130, 150, 170, 192, 135, 129):
        tokens = tiny.prompt(n, vocab, 40 + n)
        (slot,) = engine.admit(1)
        got.append(engine.step([slot], [tokens], [[n - 3, n - 1]]).float().cpu())
        engine.release([slot])
        ref.append(exact(plains, name, tokens)[[n - 3, n - 1]])
    for n in (200, 230, 250, 210):
        tokens = tiny.prompt(n, vocab, 50 + n)
        (slot,) = engine.admit(1)
        engine.step([slot], [tokens[:60]], [[]])
        got.append(engine.step([slot], [tokens[60:]], [[0, n - 61]]).float().cpu())
        engine.release([slot])
        ref.append(exact(plains, name, tokens)[[60, n - 1]])
    engine.check_errors()
    assert len(engine._prompt_graphs) >= before + 2          # both classes were recorded (and then replayed)
    check(torch.cat(got), torch.cat(ref), "float32")


@pytest.mark.parametrize("name", ["A", "M", "B"])
def test_recorded_bfloat16_steps_against_unrecorded_ones(folders, name):
    """The bfloat16 engine with recorded steps (single tokens from the second step on, prompts of a class from the second
    of the class on) against the same engine without: the same kernels on the same rows.  Recorded prompts carry rows of
    padding, which may move a product to another kernel: those are compared within the rounding of bfloat16."""
    plain_engine = model_for(folders, name, "bfloat16").engine
    recorded = model_for(folders, name, "bfloat16", use_graphs=True).engine
    vocab = tiny.ALL[name]["vocab"]
    tokens = tiny.prompt(180, vocab, 8)
    a, b = run_alone(plain_engine, tokens, [70]), run_alone(recorded, tokens, [70])
    assert len(recorded._graphs) >= 1
    assert float((a - b).abs().max()) <= 1e-6 * float(a.abs().max())
    rows = [[], []]
    for n in (140, 150, 160, 170, 145, 190):
        tokens = tiny.prompt(n, vocab, 20 + n)
        for j, engine in enumerate((plain_engine, recorded)):
            (slot,) = engine.admit(1)
            rows[j].append(engine.step([slot], [tokens], [[0, n // 2, n - 1]]).float().cpu())
            engine.release([slot])
    recorded.check_errors()
    assert len(recorded._prompt_graphs) >= 1
    a, b = torch.cat(rows[0]), torch.cat(rows[1])
    close = (a - b).abs().amax(-1) / a.abs().amax(-1)
    assert float(close.median()) < 0.02 and float((close > 0.1).double().mean()) <= 0.12


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_library(folders, plains, dtype):
    """Model.generate (scheduler, batches, recorded steps, on-device argmax) against greedy decoding: with the plain
    implementation in float32; in bfloat16 with the unrecorded engine's own logits for the same tokens, where a token that
    is not their best must be as good as the best within the noise of the format."""
    model = model_for(folders, "A", dtype, use_graphs=True)
    cfg, tensors = plains["A"]
    prompts = [tiny.prompt(n, cfg["vocab"], 60 + n) for n in (5, 37, 70)]
    outs = model.generate(prompts, max_new_tokens=12, temperature=0.0, ignore_eos=True)
    for p, o in zip(prompts, outs):
        new = list(o.tokens)
        assert len(new) == 12
        seq = list(p) + new
        if dtype == "float32":
            logits = plain.forward(seq, tensors, cfg)[0]
        else:
            logits = run_alone(model_for(folders, "A", dtype).engine, seq, [len(p)]).double()
        for j, tok in enumerate(new):
            row = logits[len(p) - 1 + j]
            best = int(row.argmax())
            if tok != best:
                gap = float(row[best] - row[tok]) / float(row.abs().max())
                assert dtype == "bfloat16" and gap < 0.03, (tok, best, gap)


def test_command_line(folders, plains, tmp_path):
    """The library's command line on a model folder (greedy tokens against the plain statement) and on random weights
    from a configuration file (its prompt and decode timings)."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, tensors = plains["C"]
    p1, p2 = tiny.prompt(6, cfg["vocab"], 1), tiny.prompt(13, cfg["vocab"], 2)
    cmd = [sys.executable, "-m", "catena_models_b200", "--model", folders["C"], "--dtype", "float32", "-n", "5",
           "--ignore-eos", "--prompt", " ".join(map(str, p1)), "--prompt", ",".join(map(str, p2))]
    run = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr
    lines = [list(map(int, l.split())) for l in run.stdout.strip().splitlines()]
    want = []
    for p in (p1, p2):
        seq = list(p)
        for _ in range(5):
            seq.append(int(plain.forward(seq, tensors, cfg)[0][-1].argmax()))
        want.append(seq[len(p):])
    assert [l[-5:] for l in lines] == want
    conf = tmp_path / "c.json"
    conf.write_text(json.dumps(tiny.TINY_M))
    bench = subprocess.run([sys.executable, "-m", "catena_models_b200", "--random", str(conf), "--bench", "--pp", "200",
                            "--tg", "6", "--tg-context", "150", "--batch", "2"], cwd=root, capture_output=True,
                           text=True, timeout=600)
    assert bench.returncode == 0, bench.stderr
    assert "pp200x2" in bench.stdout and "tg6/ctx150x2" in bench.stdout
