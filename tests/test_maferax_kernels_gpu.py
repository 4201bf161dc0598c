"""The kernels and parts that the Maferax decoder added, each against the plain statement of its mechanism
(plain_maferax.py, float64): the norm behind a sum with the average over the depth, the tanh-gelu gate, the decay of
gated linear attention in both of its forms and the scan (whole, in portions, several sequences, a slot used again),
the router with correction, groups and identity experts, and the latent attention as a part (whole, portions down to
one token, unequal sequences, pages in any order) and as a kernel with keys placed far away, at page borders, at the
row's own position and right behind it, so that a mask that is one token off changes the result beyond any tolerance."""
import types

import pytest
import torch

import plain_maferax as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def _close(got, ref, tol):
    ref = ref.to(F64).cpu()
    err = (got.to(F64).cpu() - ref).abs().max() / ref.abs().max().clamp_min(1e-9)
    assert float(err) < tol, float(err)


def _batch(lengths, starts, slots, kind=None):
    """What the kernels read of a step: sequences of `lengths` new tokens that stand at `starts`."""
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    tok_seq, tok_pos, seq_start = [], [], [0]
    for b, (n, p) in enumerate(zip(lengths, starts)):
        tok_seq += [b] * n
        tok_pos += list(range(p, p + n))
        seq_start.append(seq_start[-1] + n)
    ends = [p + n for n, p in zip(lengths, starts)]
    if kind is None:
        kind = "decode" if all(n == 1 for n in lengths) and all(p > 0 for p in starts) else "append"
    return types.SimpleNamespace(tok_seq=i32(tok_seq), tok_pos=i32(tok_pos), seq_start=i32(seq_start), seq_pos0=i32(starts),
                                 seq_end=i32(ends), seq_slot=i32(slots), B=len(lengths), T=sum(lengths), max_len=max(lengths),
                                 max_end=max(ends), positions=list(starts), lengths=list(lengths), kind=kind, shared={})


# ------------------------------------------------------------------------------ norm behind the sum, depth average
@pytest.mark.parametrize("dtype, tol", [(torch.float32, 3e-6), (torch.bfloat16, 6e-3)])
@pytest.mark.parametrize("W", [52, 256])
def test_norm_behind_the_sum_and_depth_average(dtype, tol, W):
    from catena_models_b200 import kernels

    g = torch.Generator().manual_seed(1)
    rows, depth = 37, 4
    h = torch.randn(rows, W, generator=g) * 2
    term = torch.randn(rows, W, generator=g)
    pieces = torch.randn(rows * 3, W, generator=g)
    wts = torch.rand(rows * 3, generator=g)
    w = torch.full((W,), 1.3)
    old = torch.randn(depth - 1, rows, W, generator=g)
    coef = torch.tensor([0.3, -0.2, 0.6, 0.9])
    total = 1.7 * h.double() + 0.5 * term.double() + (wts.double()[:, None] * pieces.double()).view(rows, 3, W).sum(1)
    x = plain.rms(total, 1e-5) * 1.3
    terms = kernels.Terms([(term.to(DEV), 0.5, 1), (pieces.to(DEV), 1.0, 3, None, wts.to(DEV))])
    # the sum and its norm alone
    hd = h.to(DEV).clone()
    n_out = torch.empty(rows, W, dtype=dtype, device=DEV) if dtype != torch.float32 else None
    kernels.postnorm_residual(hd, terms, 1.7, w.to(DEV), 1e-5, n_out=n_out)
    _close(hd, x, 3e-6)
    if n_out is not None:
        _close(n_out, x, tol)
    # followed by the average over what the stack held before
    hist = torch.empty(depth, rows, W, device=DEV)
    hist[:depth - 1] = old.to(DEV)
    hd = h.to(DEV).clone()
    kernels.postnorm_residual(hd, terms, 1.7, w.to(DEV), 1e-5, n_out=n_out, history=hist, coef=coef.to(DEV))
    mix = (coef.double()[:3, None, None] * old.double()).sum(0) + 0.9 * x
    _close(hist[depth - 1], x, 3e-6)
    _close(hd, mix, 3e-6)
    if n_out is not None:
        _close(n_out, mix, tol)


def test_tanh_gelu_gate():
    from catena_models_b200 import kernels

    x = torch.randn(33, 2 * 24, generator=torch.Generator().manual_seed(2)) * 2
    for dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 6e-3)):
        a = x.to(DEV, dtype).contiguous()
        ref = plain.gelu_tanh(a.double().cpu()[:, :24]) * a.double().cpu()[:, 24:]
        out = torch.empty(33, 24, dtype=dtype, device=DEV)
        kernels.swiglu(out, a, gelu=True)
        _close(out, ref, tol)


# ------------------------------------------------------------------------------ gated linear attention
@pytest.mark.parametrize("rows", [1, 8, 40, 128, 300])
def test_tanh_gelu_gate_in_the_products(rows):
    """The gate in the epilogue of the three bfloat16 products against act(g) * u of the rounded halves in float64."""
    from catena_models_b200 import kernels

    g = torch.Generator().manual_seed(rows)
    K, F = 256, 384
    x = (torch.randn(rows, K, generator=g)).to(torch.bfloat16)
    w = (torch.randn(2 * F, K, generator=g) * 0.12).to(torch.bfloat16)
    gu = (x.double() @ w.double().t()).to(torch.bfloat16).double()
    ref = plain.gelu_tanh(gu[:, :F]) * gu[:, F:]
    xd, wd = x.to(DEV), w.to(DEV)
    forms = [kernels.gemm_tc]
    if rows <= 128:
        forms.append(kernels.gemm_tc_few_rows)
    if rows <= 64:
        forms.append(kernels.gemm_skinny)
    for form in forms:
        a = torch.full((rows, F), float("nan"), dtype=torch.bfloat16, device=DEV)
        form(a, xd, wd, swiglu=2)
        torch.cuda.synchronize()
        _close(a, ref, 1e-2)
        silu = torch.empty_like(a)
        form(silu, xd, wd, swiglu=True)
        _close(silu, torch.nn.functional.silu(gu[:, :F]) * gu[:, F:], 1e-2)


@pytest.mark.parametrize("tau", [1.0, 16.0])
def test_decay_of_gated_linear_attention_both_forms(tau):
    from catena_models_b200 import kernels

    g = torch.Generator().manual_seed(3)
    rows, W, R, C = 45, 40, 6, 28
    x, w1, w2 = torch.randn(rows, W, generator=g), torch.randn(R, W, generator=g) / W ** 0.5, torch.randn(C, R, generator=g)
    b = 2.0 + torch.randn(C, generator=g)
    P = {"a1": w1.double(), "a2": w2.double(), "a2.b": b.double()}
    ref = plain.gla_decay(x.double(), P, "", {"tau": tau})
    out = torch.empty(rows, C, device=DEV)
    kernels.lowrank_decay(out, x.to(DEV), w1.to(DEV), w2.t().contiguous().to(DEV), b.to(DEV), tau=tau)
    _close(out, ref, 3e-6)
    z = (x.double() @ w1.double().T) @ w2.double().T
    kernels.decay_from_logits(out, z.float().to(DEV), b.to(DEV), tau=tau)
    _close(out, ref, 3e-6)
    # far into both tails the logarithm of the sigmoid must not lose the decay
    z = torch.tensor([[-60.0, -20.0, 0.0, 20.0, 60.0]])
    out = torch.empty(1, 5, device=DEV)
    kernels.decay_from_logits(out, z.to(DEV), torch.zeros(5, device=DEV), tau=tau)
    _close(out, torch.exp(torch.nn.functional.logsigmoid(z.double()) / tau), 3e-6)


@pytest.mark.parametrize("H, D, DV", [(2, 16, 24), (1, 12, 20), (3, 4, 12), (4, 64, 32), (2, 7, 9)])
def test_gated_scan_whole_portions_and_slots(H, D, DV):
    from catena_models_b200 import kernels

    g = torch.Generator().manual_seed(4)
    lengths = [45, 1, 70]
    T = sum(lengths)
    q, k, v, gate = (torch.randn(T, n, generator=g) for n in (H * D, H * D, H * DV, H * DV))
    decay = torch.sigmoid(2.0 + 2.0 * torch.randn(T, H * D, generator=g)) ** 0.25
    norm_w = 1 + 0.1 * torch.randn(DV, generator=g)
    eps = 1e-5

    def reference(lo, hi):
        S = torch.zeros(H, D, DV, dtype=F64)
        o = torch.zeros(hi - lo, H, DV, dtype=F64)
        for t in range(lo, hi):
            S = decay[t].double().view(H, D, 1) * S + k[t].double().view(H, D, 1) * v[t].double().view(H, 1, DV)
            o[t - lo] = torch.einsum("hdv,hd->hv", S, q[t].double().view(H, D) * D ** -0.5)
        o = plain.rms(o, eps) * norm_w.double()
        return o.reshape(hi - lo, H * DV) * plain.silu(gate[lo:hi].double())

    bounds = [0, lengths[0], lengths[0] + 1, T]
    ref = torch.cat([reference(bounds[i], bounds[i + 1]) for i in range(3)])
    state = torch.full((5, H * D * DV), float("nan"), device=DEV)
    dq, dk, dv, dg, dw = (t.to(DEV) for t in (q, k, v, gate, decay))
    nw = norm_w.repeat(H).to(DEV)

    def run(cuts, slots):
        kernels.zero_slots(state.view(1, 5, -1), slots)
        out = torch.empty(T, H * DV, device=DEV)
        at = [0, 0, 0]
        while any(at[i] < lengths[i] for i in range(3)):
            rows, lens, sl = [], [], []
            for i in range(3):
                n = min(cuts[i], lengths[i] - at[i])
                if n > 0:
                    rows += list(range(bounds[i] + at[i], bounds[i] + at[i] + n))
                    lens.append(n)
                    sl.append(slots[i])
                    at[i] += n
            idx = torch.tensor(rows, device=DEV)
            b = _batch(lens, [0] * len(lens), sl)
            o = torch.empty(len(rows), H * DV, device=DEV)
            kernels.matrix_scan("gated", o, dq[idx], dk[idx], dv[idx], dg[idx], dw[idx].contiguous(), None, nw, state, 0,
                                b.seq_start, b.seq_slot, b.B, H, D, DV, D ** -0.5, eps)
            out[idx] = o
        return out

    _close(run([1000, 1000, 1000], [0, 1, 2]), ref, 2e-5)
    _close(run([7, 1, 33], [4, 2, 0]), ref, 2e-5)            # portions; the slots of before, used again
    _close(run([2, 1, 1], [1, 0, 3]), ref, 2e-5)             # two tokens at a time, and token by token


# ------------------------------------------------------------------------------ router
@pytest.mark.parametrize("experts, identity, top, groups, scale, rows", [
    (6, 2, 3, (4, 2), 1.5, 50), (3, 0, 1, None, 1.0, 9), (1, 3, 2, (1, 1), 2.0, 70), (8, 0, 2, (2, 1), 1.0, 200),
    (5, 3, 2, (4, 2), 1.2, 33), (12, 4, 6, (8, 3), 0.7, 64)])
def test_router_with_correction_groups_and_identity(experts, identity, top, groups, scale, rows):
    """Choice, weights and the identity experts' share against the plain router.  The correction is large enough to move
    the choice away from the largest scores, and negative for some experts, so that a closed group counted as 0 instead
    of minus infinity would be chosen."""
    from catena_models_b200 import kernels

    g = torch.Generator().manual_seed(5)
    W, E = 24, experts + identity
    h = torch.randn(rows, W, generator=g)
    wr = torch.randn(E, W, generator=g) * 0.4
    corr = torch.randn(E, generator=g) * 0.3 - 0.2
    r = dict(experts=experts, top=top, identity=identity, scale=scale)
    if groups:
        r["groups"] = dict(count=groups[0], keep=groups[1])
    ids_ref, w_ref = plain.route(h.double(), {"router": wr.double(), "correction": corr.double()}, "", r)
    P = rows * top
    tile = kernels.MOE_TILE_SIMT
    ids = torch.empty(P, dtype=torch.int32, device=DEV)
    wts = torch.empty(P, dtype=torch.float32, device=DEV)
    perm = torch.empty(kernels.moe_max_tiles(P, experts, tile) * tile, dtype=torch.int32, device=DEV)
    dest = torch.empty(P, dtype=torch.int32, device=DEV)
    work = torch.empty(kernels.moe_work_size(P, experts, tile), dtype=torch.int32, device=DEV)
    tok_seq = torch.zeros(rows, dtype=torch.int32, device=DEV)
    kernels.moe_route(ids, wts, perm, dest, work, h.to(DEV), wr.to(DEV), tok_seq, top, softmax_gate=True, renormalize=True,
                      tile_rows=tile, correction=corr.to(DEV), groups=groups[0] if groups else 0, keep=groups[1] if groups else 0,
                      identity=identity, scale=scale, renorm_eps=1e-20)
    got_ids = ids.view(rows, top).cpu().long()
    got_w = wts.view(rows, top).cpu().double()
    order_ref, order_got = ids_ref.argsort(-1), got_ids.argsort(-1)
    assert torch.equal(ids_ref.gather(1, order_ref), got_ids.gather(1, order_got))
    _close(got_w.gather(1, order_got), w_ref.gather(1, order_ref), 2e-5)
    # identity experts get no row of the grouped products; real experts do
    d = dest.view(rows, top).cpu()
    assert bool(((d < 0) == (got_ids >= experts)).all())
    if identity:
        same = torch.empty(rows, W, device=DEV)
        kernels.moe_identity(same, h.to(DEV), ids, wts, top, experts)
        share = (w_ref * (ids_ref >= experts)).sum(-1, keepdim=True)
        _close(same, share * h.double(), 2e-5)


# ------------------------------------------------------------------------------ latent attention
def _latent_case(seed, H, D, R, DV, KR, QR, W, rot_dims, base=1000.0, scale=0.3):
    g = torch.Generator().manual_seed(seed)
    n = lambda *s: torch.randn(*s, generator=g) / s[-1] ** 0.5
    p = "m."
    P = {p + "dq": n(QR, W), p + "dq.norm": 1 + 0.1 * torch.randn(QR, generator=g), p + "uq": n(H * (D + R), QR) * 2,
         p + "dkv": n(KR + R, W), p + "dkv.norm": 1 + 0.1 * torch.randn(KR, generator=g), p + "uk": n(H * D, KR) * 2,
         p + "uv": n(H * DV, KR), p + "g": n(H, W) * 2, p + "o": n(W, H * DV)}
    m = dict(heads=H, dim=D, rot_dim=R, vdim=DV, kv_rank=KR, q_rank=QR, scale=scale, rot=dict(dims=rot_dims, base=base))
    return P, m


def _latent_part(P, m, W, dtype):
    from catena_models_b200.engine.runtime import Runtime
    from catena_models_b200.parts import build_part

    rt = Runtime(dtype, DEV)
    pos = build_part("position", "paired_rotary", dims=m["rot"]["dims"], theta=m["rot"]["base"])
    part = build_part("mixer", "latent_attention", prefix="m.", hidden=W, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"],
                      value_dim=m["vdim"], kv_rank=m["kv_rank"], q_rank=m["q_rank"], position=pos, scale=m["scale"], eps=1e-5,
                      out_dtype="float32")
    part.bind_all({k: v.to(DEV, dtype if v.dim() == 2 else torch.float32) for k, v in P.items()}, rt)
    return rt, part


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 2e-5), (torch.bfloat16, 2.5e-2)])
@pytest.mark.parametrize("H, D, R, DV, KR, QR, W, rot_dims", [
    (3, 16, 8, 24, 40, 24, 64, 8), (1, 12, 6, 20, 21, 10, 36, 4), (2, 8, 2, 8, 16, 16, 32, 2), (4, 32, 16, 64, 64, 48, 128, 16),
    (5, 8, 4, 8, 136, 8, 40, 4)])
def test_latent_attention_part_whole_portions_and_pages(dtype, tol, H, D, R, DV, KR, QR, W, rot_dims):
    """The mixer over a paged cache whose pages lie in any order: three unequal sequences as whole prompts, in portions
    down to one token (the single-token steps take the form that cuts the keys into runs), and with slots used again."""
    from catena_models_b200.cache.spec import KVStateSpec

    P, m = _latent_case(6, H, D, R, DV, KR, QR, W, rot_dims)
    if dtype == torch.bfloat16:
        P = {k: v.to(torch.bfloat16).float() for k, v in P.items()}
    rt, part = _latent_part(P, m, W, dtype)
    g = torch.Generator().manual_seed(7)
    lengths = [150, 3, 70]
    xs = [torch.randn(n, W, generator=g) for n in lengths]
    if dtype == torch.bfloat16:
        xs = [x.to(torch.bfloat16).float() for x in xs]
    P64 = {k: v.double() for k, v in P.items()}
    refs = [plain.latent_attention(x.double(), P64, "m.", m, 1e-5)[0] for x in xs]
    spec = part.state_spec()
    assert spec == KVStateSpec(1, -(-(KR + R) // 8) * 8, 0, planes=1)
    pages_per, slots_n = 3, 6
    pool = torch.full((1, slots_n * pages_per + 1, 1, 64, spec.head_dim), float("nan"), dtype=dtype, device=DEV)
    ptab = torch.randperm(slots_n * pages_per, generator=g).view(slots_n, pages_per).to(DEV, torch.int32)
    state = types.SimpleNamespace(pool=pool, ptab=ptab, spec=spec)

    def run(cuts, slots):
        outs = [torch.empty(n, W) for n in lengths]
        at = [0, 0, 0]
        while any(at[i] < lengths[i] for i in range(3)):
            rows, lens, starts, sl, who = [], [], [], [], []
            for i in range(3):
                n = min(cuts[i], lengths[i] - at[i])
                if n > 0:
                    rows.append(xs[i][at[i]:at[i] + n])
                    lens.append(n); starts.append(at[i]); sl.append(slots[i]); who.append(i)
                    at[i] += n
            b = _batch(lens, starts, sl)
            y = part.forward(rt, b, torch.cat(rows).to(DEV, dtype), state).float().cpu()
            o = 0
            for i, n, s in zip(who, lens, starts):
                outs[i][s:s + n] = y[o:o + n]
                o += n
        return outs

    for cuts, slots in (([1000] * 3, [0, 1, 2]), ([7, 1, 33], [4, 2, 0]), ([64, 2, 1], [1, 5, 3]), ([149, 1, 1], [2, 0, 4])):
        for got, ref in zip(run(cuts, slots), refs):
            _close(got, ref, tol)


@pytest.mark.parametrize("H, D, R, DV, KR, QR, W, rot_dims, head", [
    (4, 32, 16, 64, 64, 48, 128, 16, 64), (2, 64, 32, 48, 128, 40, 96, 32, 128), (3, 24, 8, 128, 72, 24, 64, 6, 128),
    (1, 16, 2, 16, 16, 16, 32, 2, 64)])
def test_latent_attention_expanded_prompt_form(H, D, R, DV, KR, QR, W, rot_dims, head):
    """Whole prompts in bfloat16, long enough for the tensor-core attention kernels of both kinds: the form that expands the
    step's latents into keys and values per head against the form that reads the cache with the products moved to the
    query side, and both against the plain statement.  Afterwards single tokens go on from the cache that the expanded
    form's step wrote."""
    from catena_models_b200 import kernels

    P, m = _latent_case(11, H, D, R, DV, KR, QR, W, rot_dims)
    P = {k: v.to(torch.bfloat16).float() for k, v in P.items()}
    rt, part = _latent_part(P, m, W, torch.bfloat16)
    assert part.expand_head == head
    g = torch.Generator().manual_seed(12)
    lengths = [1100, 65, 300]
    xs = [torch.randn(n + 2, W, generator=g).to(torch.bfloat16).float() for n in lengths]
    P64 = {k: v.double() for k, v in P.items()}
    refs = [plain.latent_attention(x.double(), P64, "m.", m, 1e-5)[0] for x in xs]
    spec = part.state_spec()
    pages_per, slots_n = 18, 3
    ptab = torch.randperm(slots_n * pages_per, generator=g).view(slots_n, pages_per).to(DEV, torch.int32)
    outs = {}
    for form, least in (("expanded", 64), ("cache", 1 << 30)):
        part.expand_min_tokens = least
        pool = torch.full((1, slots_n * pages_per + 1, 1, 64, spec.head_dim), float("nan"), dtype=torch.bfloat16, device=DEV)
        state = types.SimpleNamespace(pool=pool, ptab=ptab, spec=spec)
        names = []
        with kernels.Timeline() as tl:
            y = part.forward(rt, _batch(lengths, [0, 0, 0], [2, 0, 1], kind="prefill"),
                             torch.cat([x[:n] for x, n in zip(xs, lengths)]).to(DEV, torch.bfloat16), state).float().cpu()
        names = [r["name"] for r in tl.rows()]
        assert ("latent_expand" in names) == (form == "expanded") and ("latent_attn" in names) == (form == "cache"), names
        outs[form] = y
        o = 0
        for n, ref in zip(lengths, refs):
            _close(y[o:o + n], ref[:n], 4e-2)
            o += n
        # two more tokens each, one at a time, over what the step left in the cache
        for k in range(2):
            b = _batch([1, 1, 1], [n + k for n in lengths], [2, 0, 1], kind="decode")
            y1 = part.forward(rt, b, torch.stack([x[n + k] for x, n in zip(xs, lengths)]).to(DEV, torch.bfloat16), state).float().cpu()
            for i, (n, ref) in enumerate(zip(lengths, refs)):
                _close(y1[i:i + 1], ref[n + k:n + k + 1], 2.5e-2)
    _close(outs["expanded"], outs["cache"], 2e-2)


@pytest.mark.parametrize("H, R, KR, positions", [
    (5, 6, 21, [0, 1, 31, 32, 200]), (16, 16, 128, [63, 64, 700, 3, 1023]), (20, 8, 136, [500, 33]), (33, 32, 512, [90, 600, 2]),
    (1, 2, 8, [15, 16, 17]), (12, 0, 64, [300])])
def test_latent_attention_single_tokens_on_the_tensor_cores(H, R, KR, positions):
    """One token per sequence over a bfloat16 cache: the tensor-core form against the float64 sum over the same entries
    and queries (both rounded to bfloat16 beforehand, so that only the weights' rounding remains), with the keys in one
    run and cut into runs, a gate, heads that do not fill a block of 16, latents that do not fill the warps' channels,
    pages in any order and used pages that hold other values past each sequence's end."""
    from catena_models_b200 import kernels

    E, EC = KR + R, -(-(KR + R) // 8) * 8
    B = len(positions)
    g = torch.Generator().manual_seed(21)
    per = -(-(max(positions) + 1) // 64)
    order = torch.randperm(B * per + 2, generator=g)[:B * per].view(B, per)
    ptab = order.to(DEV, torch.int32)
    pool = torch.full((1, B * per + 2, 1, 64, EC), 30.0, dtype=torch.bfloat16, device=DEV)
    entries = []
    for b, pos in enumerate(positions):
        lat = (torch.randn(pos + 1, E, generator=g) * 0.5).to(torch.bfloat16)
        entries.append(lat.double())
        for p in range(pos + 1):
            pool[0, order[b, p // 64], 0, p % 64, :E] = lat[p].to(DEV)
            pool[0, order[b, p // 64], 0, p % 64, E:] = 0
    qa = (torch.randn(B, H, E, generator=g) * 0.4).to(torch.bfloat16).float()
    gate = torch.randn(B, H + 3, generator=g).to(torch.bfloat16)
    scale = 0.7
    ref = torch.stack([torch.softmax(torch.einsum("he,ne->hn", qa[b].double(), entries[b]) * scale, -1) @ entries[b][:, :KR]
                       * torch.sigmoid(gate[b, :H].double())[:, None] for b in range(B)])
    batch = _batch([1] * B, positions, list(range(B)), kind="decode")
    for keys in (None, 1024, 64):
        splits, chunk, parts = 1, 0, None
        if keys:
            splits, chunk = kernels.latent_attn_splits(B, H, keys, heads_per_block=16)
            parts = torch.full((B * H * splits * (2 + KR),), float("nan"), device=DEV)
        out = torch.full((B, H * KR), float("nan"), device=DEV)
        kernels.latent_attn(out, qa.reshape(B, H * E).to(DEV), gate.to(DEV), pool, ptab, batch, H, R, KR, scale, splits=splits,
                            chunk=chunk, parts=parts, tensor_cores=True)
        _close(out.view(B, H, KR), ref, 6e-3)
        plain_out = torch.full((B, H * KR), float("nan"), device=DEV)
        kernels.latent_attn(plain_out, qa.reshape(B, H * E).to(DEV), gate.to(DEV), pool, ptab, batch, H, R, KR, scale, splits=splits,
                            chunk=chunk, parts=parts)
        _close(plain_out.view(B, H, KR), ref, 2e-5)


@pytest.mark.parametrize("decode", [False, True, "tensor cores"])
def test_latent_attention_keys_far_away_at_borders_and_behind_the_row(decode):
    """One key is made to stand out (a query and a latent row scaled along one direction) so that the sum over the
    latents is that key's row if and only if the row sees it: keys at position 0 and 3 from far away, on both sides of
    page borders, at the row's own position; a key right behind the row, and what a used page holds past the sequence's
    end, must stay unseen."""
    from catena_models_b200 import kernels

    H, R, KR = 3, 8, 40
    E, EC = KR + R, 48
    n = 700
    g = torch.Generator().manual_seed(8)
    lat = torch.randn(n + 64, E, generator=g) * 0.3
    pages = -(-(n + 64) // 64)
    order = torch.randperm(pages + 3, generator=g)[:pages].tolist()
    ptab = torch.full((2, pages), -1, dtype=torch.int32, device=DEV)
    ptab[1] = torch.tensor(order, dtype=torch.int32)
    cases = []        # (row position, loud key, seen?)
    for row, key in ((699, 0), (699, 3), (650, 63), (650, 64), (128, 127), (128, 128), (300, 300), (64, 63), (64, 64), (1, 0), (0, 0)):
        cases.append((row, key, True))
    for row, key in ((63, 64), (127, 128), (300, 301), (0, 1), (650, 699)):
        cases.append((row, key, False))
    for row, key, seen in cases:
        direction = torch.randn(E, generator=g)
        direction /= direction.norm()
        keys = lat.clone()
        keys[key] += 8.0 * direction
        mma = decode == "tensor cores"
        if mma:
            keys = keys.to(torch.bfloat16).float()
        pool = torch.full((1, pages + 3, 1, 64, EC), 50.0, device=DEV, dtype=torch.bfloat16 if mma else torch.float32)       # what other sequences left in the pages
        for p in range(n + 64 if not decode else row + 1):
            pool[0, order[p // 64], 0, p % 64, :E] = keys[p].to(DEV)
            if mma:
                pool[0, order[p // 64], 0, p % 64, E:] = 0
        qa = torch.randn(1, H, E, generator=g) * 0.3
        qa[0, 1] += 8.0 * direction                   # head 1 looks for the loud key; the others do not
        if mma:
            qa = qa.to(torch.bfloat16).float()
        if decode:
            b = _batch([1], [row], [1], kind="decode") if row > 0 or mma else _batch([1], [0], [1], kind="prefill")
            rows = qa
        else:
            # a prompt step of the rows row - 2 .. row + 1 standing on older entries; the row in question is one of them
            first = max(0, row - 2)
            b = _batch([row + 2 - first], [first], [1])
            rows = torch.randn(b.T, H, E, generator=g) * 0.3
            rows[row - first] = qa[0]
        out = torch.empty(b.T, H * KR, device=DEV)
        splits, chunk, parts = 1, 0, None
        if decode:
            splits, chunk = kernels.latent_attn_splits(1, H, 1024)
            assert splits > 1
            parts = torch.full((H * splits * (2 + KR),), float("nan"), device=DEV)
        kernels.latent_attn(out, rows.reshape(b.T, H * E).to(DEV), None, pool, ptab, b, H, R, KR, 1.0, splits=splits, chunk=chunk,
                            parts=parts, tensor_cores=mma)
        at = 0 if decode else row - max(0, row - 2)
        s = torch.einsum("he,ne->hn", qa[0].double(), keys[:row + 1].double())
        ref = torch.softmax(s, -1) @ keys[:row + 1, :KR].double()
        _close(out[at].view(H, KR), ref, 6e-3 if mma else 2e-5)
        loud = float(torch.softmax(s, -1)[1, key]) if key <= row else 0.0
        assert (loud > 0.9) == seen, (row, key, loud)
