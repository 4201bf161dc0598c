"""The Maferax decoder in the engine against the plain implementation (plain_maferax.py): every mechanism in a
model of its own, whole prompts, prompts against token-by-token decoding, portions down to two tokens, unequal
batches against each request alone, slots and pages that are used again, decoding across page borders, the first
tokens, other sizes (one head, one expert per token, a turned part that is only partly turned, a layer without
feed-forward), recorded steps, and greedy generation through the library's own entry point."""
import pytest
import torch

import plain_maferax as plain
import tiny_maferax as tiny

pytestmark = pytest.mark.gpu

TOL_F32 = 3e-5            # largest |engine - plain| relative to the largest |logit| of the row: float32 sums against float64
# bfloat16: a row's error relative to the row's largest logit.  The yardstick is the plain implementation with roundings
# to bfloat16 where an engine stores activations: its distance from the exact result is what the storage format alone
# costs on this input.  The engine's typical row must be as close as the yardstick's (twice its median) and few rows
# may lie far beyond the yardstick's 90th percentile.  The exact result uses the yardstick's choice of experts, so that a
# close call of a router that rounding turns does not count as an error of the arithmetic.
BF16_FACTOR, BF16_SLACK, BF16_ROWS_OVER = 2.0, 0.004, 0.1


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("maferax")
    return {name: tiny.make_folder(tmp, name, seed=40 + i) for i, name in enumerate(tiny.ALL)}


@pytest.fixture(scope="module")
def plains(folders):
    return {name: tiny.load_plain(f) for name, f in folders.items()}


_models = {}


def model_for(folders, name, dtype, **kw):
    from catena_models_b200.api import Model

    key = (name, dtype, tuple(sorted(kw.items())))
    if key not in _models:
        _models[key] = Model.load(folders[name], dtype=dtype, max_tokens=4096, **kw)
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


def exact(plains, name, tokens, dtype="float32"):
    cfg, tensors = plains[name]
    if dtype == "bfloat16":
        ids = {}
        same = plain.forward(tokens, tensors, cfg, rd=plain.to_bf16, ids_out=ids)[0]
        return plain.forward(tokens, tensors, cfg, expert_ids=ids)[0], same
    return plain.forward(tokens, tensors, cfg)[0]


def run_alone(engine, tokens, cuts):
    """One request through the engine in steps of the given sizes (the rest token by token); every logit."""
    (slot,) = engine.admit(1)
    out, at = [], 0
    try:
        for n in list(cuts) + [1] * len(tokens):
            if at >= len(tokens):
                break
            part = tokens[at:at + n]
            out.append(engine.step([slot], [part], [list(range(len(part)))]).float().cpu())
            at += len(part)
        engine.check_errors()
    finally:
        engine.release([slot])
    return torch.cat(out)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tiny.ALL))
def test_whole_prompt(folders, plains, name, dtype):
    engine = model_for(folders, name, dtype).engine
    tokens = tiny.prompt(150, tiny.ALL[name]["vocab"], 1)
    check(run_alone(engine, tokens, [len(tokens)]), exact(plains, name, tokens, dtype), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "M", "latent", "gla", "moe"])
def test_prompt_then_token_by_token(folders, plains, name, dtype):
    """A prompt in one step, then tokens one by one (recorded decode steps from the second on): across a page
    border (64) and from the very first token on."""
    engine = model_for(folders, name, dtype).engine
    tokens = tiny.prompt(140, tiny.ALL[name]["vocab"], 2)
    ref = exact(plains, name, tokens, dtype)
    check(run_alone(engine, tokens, [50]), ref, dtype)
    check(run_alone(engine, tokens, [1]), ref, dtype)


@pytest.mark.parametrize("name", ["A", "B", "C", "M"])
def test_portions_of_several_sizes(folders, plains, name):
    engine = model_for(folders, name, "float32").engine
    tokens = tiny.prompt(200, tiny.ALL[name]["vocab"], 3)
    ref = exact(plains, name, tokens)
    for cuts in ([2] * 100, [3, 61, 1, 64, 2, 69], [64, 64, 64, 8], [127, 2, 2, 69], [1, 1, 2, 5, 7, 100, 84]):
        check(run_alone(engine, tokens, cuts), ref, "float32")
    bf = model_for(folders, name, "bfloat16").engine
    check(run_alone(bf, tokens, [33, 2, 65, 100]), exact(plains, name, tokens, "bfloat16"), "bfloat16")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "M"])
def test_unequal_batch_against_each_alone(folders, plains, name, dtype):
    """Four requests of unequal length start together and are decoded together; the shorter ones end earlier and
    their slots and pages are taken by new requests while the others go on."""
    engine = model_for(folders, name, dtype).engine
    vocab = tiny.ALL[name]["vocab"]
    lens, extra = [1, 70, 23, 131], [3, 9, 30, 12]
    toks = [tiny.prompt(n + e, vocab, 10 + i) for i, (n, e) in enumerate(zip(lens, extra))]
    refs = [exact(plains, name, t, dtype) for t in toks]
    slots = engine.admit(4)
    got = [[] for _ in toks]
    logits = engine.step(slots, [t[:n] for t, n in zip(toks, lens)], [list(range(n)) for n in lens]).float().cpu()
    at = 0
    for i, n in enumerate(lens):
        got[i].append(logits[at:at + n])
        at += n
    live, pos = list(range(4)), list(lens)
    late = None
    while live:
        logits = engine.step([slots[i] for i in live], [[toks[i][pos[i]]] for i in live]).float().cpu()
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
            late = engine.step([s], [late_tokens], [list(range(40))]).float().cpu()
            engine.release([s])
    engine.check_errors()
    for i in range(4):
        check(torch.cat(got[i]), refs[i], dtype)
    check(late, exact(plains, name, late_tokens, dtype), dtype)


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
    engine = model_for(folders, name, "float32").engine
    tokens = tiny.prompt(400, tiny.ALL[name]["vocab"], 4)
    check(run_alone(engine, tokens, [5]), exact(plains, name, tokens), "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "M"])
def test_recorded_prompt_classes(folders, plains, name, dtype):
    """Prompts of one class of shapes (rows rounded up to 64, the same number of wanted places) run as a replayed
    recording from the third on, with rows of padding behind the tokens; so do portions on top of held tokens."""
    engine = model_for(folders, name, dtype).engine
    vocab = tiny.ALL[name]["vocab"]
    before = len(engine._prompt_graphs)
    got, ref = [], []
    for n in (130, 150, 170, 192, 135, 129):
        tokens = tiny.prompt(n, vocab, 40 + n)
        (slot,) = engine.admit(1)
        got.append(engine.step([slot], [tokens], [[n - 3, n - 1]]).float().cpu())
        engine.release([slot])
        full = exact(plains, name, tokens, dtype)
        ref.append(tuple(f[[n - 3, n - 1]] for f in full) if isinstance(full, tuple) else full[[n - 3, n - 1]])
    for n in (200, 230, 250, 210):
        tokens = tiny.prompt(n, vocab, 50 + n)
        (slot,) = engine.admit(1)
        engine.step([slot], [tokens[:60]], [[]])
        got.append(engine.step([slot], [tokens[60:]], [[0, n - 61]]).float().cpu())
        engine.release([slot])
        full = exact(plains, name, tokens, dtype)
        ref.append(tuple(f[[60, n - 1]] for f in full) if isinstance(full, tuple) else full[[60, n - 1]])
    engine.check_errors()
    assert len(engine._prompt_graphs) >= before + 2          # both classes were recorded (and then replayed)
    merged = tuple(torch.cat([r[i] for r in ref]) for i in range(2)) if isinstance(ref[0], tuple) else torch.cat(ref)
    check(torch.cat(got), merged, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_library(folders, plains, dtype):
    """Model.generate (scheduler, batches, on-device argmax) against greedy decoding with the plain implementation."""
    model = model_for(folders, "A", dtype)
    cfg, tensors = plains["A"]
    prompts = [tiny.prompt(n, cfg["vocab"], 60 + n) for n in (5, 37, 70)]
    outs = model.generate(prompts, max_new_tokens=12, temperature=0.0, ignore_eos=True)
    for p, o in zip(prompts, outs):
        new = list(o.tokens)
        assert len(new) == 12
        seq = list(p)
        for tok in new:
            logits = plain.forward(seq, tensors, cfg)[0][-1]
            best = int(logits.argmax())
            if tok != best:
                # bfloat16 may turn a close call the other way: the token it chose must be as good as the best within its noise
                gap = float(logits[best] - logits[tok]) / float(logits.abs().max())
                assert dtype == "bfloat16" and gap < 0.03, (tok, best, gap)
            seq.append(tok)
