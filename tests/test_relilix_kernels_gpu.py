"""The mechanisms that the Relilix decoder added, each alone against the plain statement (plain_relilix.py) or a float64
sum written here: capped scores in every form of the attention kernels (whole prompts on the CUDA cores, mma.sync and
tcgen05; single tokens on the CUDA cores and mma.sync; portions on top of a paged cache in all three forms), with a key
that decides the row from far away, just inside and just outside the window; the taps with interleaved rotation, values
taken from the keys and a ring of pages, whole, token by token and in portions; the rescaled interleaved rotation's
magnitude in the latent attention and a layer that reads another layer's latents; the router's groups scored by their
two best; the clamped gate alone, in the grouped products and in a dense feed-forward."""
import math
import types

import pytest
import torch

import plain_relilix as plain
from test_kernels_gpu import DEV, _paged_cache, close, rnd

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from catena_models_b200 import kernels
    kernels.lib()
    return kernels


def capped_attention(q, k, v, window, scale, cap, first=0):
    """float64: rows `first`.. of softmax(cap tanh(q k^T scale / cap)) v over the keys j <= i, i - j < window.
    q [T, QH, HD], k and v [T, KVH, HD]."""
    T, QH, HD = q.shape
    KVH = k.shape[1]
    pos = torch.arange(T)
    hidden = pos[None, :] > pos[:, None]
    if window > 0:
        hidden |= pos[None, :] + window <= pos[:, None]
    out = torch.zeros(T, QH, HD, dtype=torch.float64)
    for h in range(QH):
        g = h // (QH // KVH)
        s = (q[:, h].double() @ k[:, g].double().T) * scale
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        out[:, h] = torch.softmax(s.masked_fill(hidden, -math.inf), -1) @ v[:, g].double()
    return out[first:]


def _rows(T, QH, KVH, HD, dtype, seed, spread=2.5):
    """Packed rows [q | k | v] whose scores spread well beyond a cap of 2."""
    buf = rnd(T, (QH + 2 * KVH) * HD, dtype=dtype, scale=1.0, seed=seed)
    buf[:, :QH * HD] *= spread
    return buf, buf[:, :QH * HD], buf[:, QH * HD:(QH + KVH) * HD], buf[:, (QH + KVH) * HD:]


def _views(q, k, v, QH, KVH, HD):
    T = q.shape[0]
    return q.float().cpu().view(T, QH, HD), k.float().cpu().view(T, KVH, HD), v.float().cpu().view(T, KVH, HD)


# ------------------------------------------------------------------------------------------ whole prompts
@pytest.mark.parametrize("cap", [2.0, 40.0])
@pytest.mark.parametrize("impl, dtype, QH, KVH, HD, T, window", [
    ("simt", torch.float32, 4, 2, 24, 150, 37), ("simt", torch.bfloat16, 3, 1, 40, 130, 0), ("simt", torch.float32, 2, 2, 16, 90, 3),
    ("mma", torch.bfloat16, 4, 2, 64, 300, 100), ("mma", torch.bfloat16, 2, 1, 112, 200, 0), ("mma", torch.bfloat16, 6, 6, 16, 140, 64),
    ("tc", torch.bfloat16, 4, 2, 64, 900, 0), ("tc", torch.bfloat16, 2, 1, 128, 1000, 800), ("tc", torch.bfloat16, 2, 2, 64, 700, 130)])
def test_capped_scores_in_prompt_attention(K, impl, dtype, QH, KVH, HD, T, window, cap):
    """Random rows whose raw scores reach several times a cap of 2, or a quarter of a cap of 40 (where the tensor-core kernels
    form the tanh of most rows by its series): the result follows the capped scores, not the raw ones."""
    if cap > 2.0 and impl == "simt":
        pytest.skip("one form of the tanh")
    scale = HD ** -0.5
    _, q, k, v = _rows(T, QH, KVH, HD, dtype, 3)
    lens = [T - 70, 70]                                # two sequences side by side
    starts = torch.tensor([0, lens[0], T], dtype=torch.int32, device=DEV)
    ctx = torch.empty(T, QH * HD, dtype=dtype, device=DEV)
    if impl == "tc":
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        K.attn_prefill_tc(ctx, q, k, v, None, starts, 2, max(lens), QH, KVH, HD, window, scale, err=err, softcap=cap)
        assert int(err) == 0
    else:
        fn = K.attn_prefill_mma if impl == "mma" else K.attn_prefill_simt
        fn(ctx, q, k, v, None, starts, 2, max(lens), QH, KVH, HD, window, scale, softcap=cap)
    qv, kv, vv = _views(q, k, v, QH, KVH, HD)
    ref = torch.cat([capped_attention(qv[a:b], kv[a:b], vv[a:b], window, scale, cap) for a, b in ((0, lens[0]), (lens[0], T))])
    close(ctx.view(T, QH, HD), ref, dtype)
    raw = torch.cat([capped_attention(qv[a:b], kv[a:b], vv[a:b], window, scale, 0.0) for a, b in ((0, lens[0]), (lens[0], T))])
    assert float((ref - raw).abs().max()) > (0.2 if cap == 2.0 else 0.02)           # the cap matters on this input


@pytest.mark.parametrize("impl, dtype, HD, T", [("simt", torch.float32, 32, 400), ("mma", torch.bfloat16, 64, 400),
                                                ("tc", torch.bfloat16, 64, 900), ("tc", torch.bfloat16, 128, 900)])
@pytest.mark.parametrize("window", [0, 200])
def test_a_far_key_under_the_cap_and_the_windows_edge_in_prompts(K, impl, dtype, HD, T, window):
    """One key is made to stand out (its capped score is the cap itself); exactly the queries whose window holds it
    return its value: the one at its own position first, the one window - 1 later last."""
    QH, KVH, cap, far = 2, 1, 15.0, 130
    buf = rnd(T, (QH + 2 * KVH) * HD, dtype=dtype, scale=0.3, seed=11)
    q, k, v = buf[:, :QH * HD], buf[:, QH * HD:(QH + KVH) * HD], buf[:, (QH + KVH) * HD:]
    k[far] = 0
    k[far, 0] = 30.0
    q[:, 0] = 30.0                                     # every query of head 0 looks for it
    starts = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    ctx = torch.empty(T, QH * HD, dtype=dtype, device=DEV)
    scale = HD ** -0.5
    if impl == "tc":
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        K.attn_prefill_tc(ctx, q, k, v, None, starts, 1, T, QH, KVH, HD, window, scale, err=err, softcap=cap)
        assert int(err) == 0
    else:
        fn = K.attn_prefill_mma if impl == "mma" else K.attn_prefill_simt
        fn(ctx, q, k, v, None, starts, 1, T, QH, KVH, HD, window, scale, softcap=cap)
    close(ctx.view(T, QH, HD), capped_attention(*_views(q, k, v, QH, KVH, HD), window, scale, cap), dtype)
    hit = (ctx.view(T, QH, HD)[:, 0].float() - v[far].float()).abs().max(dim=-1).values < 0.05
    expect = torch.arange(T, device=DEV) >= far
    if window:
        expect &= torch.arange(T, device=DEV) < far + window
    assert torch.equal(hit, expect)


# ------------------------------------------------------------------------------------------ single tokens
@pytest.mark.parametrize("dtype, tensor_cores, cap", [(torch.float32, False, 2.0), (torch.bfloat16, False, 2.0), (torch.bfloat16, True, 2.0),
                                                      (torch.bfloat16, True, 40.0)])
@pytest.mark.parametrize("QH, KVH, HD, window", [(4, 2, 16, 0), (6, 3, 128, 90), (5, 5, 32, 70), (8, 2, 64, 300), (2, 1, 48, 0)])
def test_capped_scores_in_single_token_attention(K, dtype, tensor_cores, cap, QH, KVH, HD, window):
    K.set_decode_attention_tensor_cores(tensor_cores)
    try:
        ring = (window + 63) // 64 * 64 if window else 0
        lens, scale, n_chunks = [1, 64, 65, 300, 700], HD ** -0.5, 4
        g = torch.Generator().manual_seed(HD + window)
        kv = [torch.randn(n, 2, KVH, HD, generator=g) for n in lens]
        pool, pages, ptab = _paged_cache(K, kv, KVH, HD, dtype, lens, ring)
        B = len(lens)
        q = rnd(B, QH * HD, dtype=dtype, scale=2.5, seed=7)
        pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
        slots = torch.arange(1, B + 1, dtype=torch.int32, device=DEV)
        part_o, part_ml = K.attn_decode_scratch(B, QH, HD, n_chunks, DEV)
        ctx = torch.full((B, QH * HD), float("nan"), dtype=dtype, device=DEV)
        K.attn_decode(ctx, q, None, pos, slots, pool, pages, ptab, ring, window, QH, KVH, HD, n_chunks, scale, part_o, part_ml,
                      softcap=cap)
        moved = 0.0
        for b, n in enumerate(lens):
            kk, vv = kv[b][:, 0].to(dtype).float(), kv[b][:, 1].to(dtype).float()
            qq = torch.zeros(n, QH, HD)
            qq[-1] = q[b].float().cpu().view(QH, HD)
            ref = capped_attention(qq, kk, vv, window, scale, cap, first=n - 1)[0]
            close(ctx[b].view(QH, HD), ref, dtype)
            moved = max(moved, float((ref - capped_attention(qq, kk, vv, window, scale, 0.0, first=n - 1)[0]).abs().max()))
        assert moved > (0.2 if cap == 2.0 else 0.02)
    finally:
        K.set_decode_attention_tensor_cores(True)


@pytest.mark.parametrize("dtype, tensor_cores", [(torch.float32, False), (torch.bfloat16, True)])
def test_a_far_key_under_the_cap_and_the_windows_edge_in_single_tokens(K, dtype, tensor_cores):
    """The key that stands out is found among hundreds while the window holds it (also in the last entry that it holds)
    and is invisible one token later, in a ring that has turned over."""
    K.set_decode_attention_tensor_cores(tensor_cores)
    try:
        QH = KVH = 1
        HD, n, cap = 16, 500, 15.0
        for window, far, seen in [(0, 3, True), (200, n - 200, True), (200, n - 201, False), (88, n - 88, True), (88, n - 89, False)]:
            ring = (window + 63) // 64 * 64 if window else 0
            kv = [torch.randn(n, 2, KVH, HD, generator=torch.Generator().manual_seed(1)) * 0.1]
            kv[0][far, 0, 0] = 0.0
            kv[0][far, 0, 0, 0] = 40.0
            kv[0][far, 1, 0] = 7.0
            pool, pages, ptab = _paged_cache(K, kv, KVH, HD, dtype, [n], ring)
            q = torch.zeros(1, HD, dtype=dtype, device=DEV)
            q[0, 0] = 40.0
            pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
            slots = torch.tensor([1], dtype=torch.int32, device=DEV)
            part_o, part_ml = K.attn_decode_scratch(1, QH, HD, 2, DEV)
            ctx = torch.empty(1, HD, dtype=dtype, device=DEV)
            K.attn_decode(ctx, q, None, pos, slots, pool, pages, ptab, ring, window, QH, KVH, HD, 2, HD ** -0.5, part_o, part_ml,
                          softcap=cap)
            if seen:
                assert torch.allclose(ctx.float().cpu(), torch.full((1, HD), 7.0), atol=5e-2), (window, far)
            else:
                assert float(ctx.float().abs().max()) < 1.0, (window, far)
    finally:
        K.set_decode_attention_tensor_cores(True)


# ------------------------------------------------------------------------------------------ portions on top of a cache
@pytest.mark.parametrize("impl, dtype, QH, KVH, HD, window", [("simt", torch.float32, 4, 2, 24, 50), ("mma", torch.bfloat16, 4, 2, 64, 0),
                                                              ("mma", torch.bfloat16, 2, 1, 128, 90), ("tc", torch.bfloat16, 4, 1, 64, 600),
                                                              ("tc", torch.bfloat16, 2, 2, 128, 0)])
def test_capped_scores_in_portions_on_top_of_held_tokens(K, impl, dtype, QH, KVH, HD, window):
    past, new, cap, scale = [0, 700, 65], [40, 130, 200], 2.0, HD ** -0.5
    ring = (window + 63) // 64 * 64 if window else 0
    g = torch.Generator().manual_seed(5)
    seqs = [torch.randn(p + n, 3, max(QH, KVH), HD, generator=g) for p, n in zip(past, new)]
    for s in seqs:
        s[:, 0] *= 2.5
    kv = [s[:p, 1:, :KVH] for s, p in zip(seqs, past)]
    pool, pages, ptab = _paged_cache(K, kv, KVH, HD, dtype, past, ring)
    T = sum(new)
    buf = torch.empty(T, (QH + 2 * KVH) * HD, dtype=dtype, device=DEV)
    at = 0
    for s, p, n in zip(seqs, past, new):
        buf[at:at + n, :QH * HD] = s[p:, 0, :QH].reshape(n, -1).to(dtype)
        buf[at:at + n, QH * HD:(QH + KVH) * HD] = s[p:, 1, :KVH].reshape(n, -1).to(dtype)
        buf[at:at + n, (QH + KVH) * HD:] = s[p:, 2, :KVH].reshape(n, -1).to(dtype)
        at += n
    q, k, v = buf[:, :QH * HD], buf[:, QH * HD:(QH + KVH) * HD], buf[:, (QH + KVH) * HD:]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    starts, pos0, slots = i32([0, new[0], new[0] + new[1], T]), i32(past), i32([1, 2, 3])
    ctx = torch.empty(T, QH * HD, dtype=dtype, device=DEV)
    if impl == "tc":
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        K.attn_append_tc(ctx, q, k, v, None, starts, pos0, slots, pool, pages, ptab, ring, 3, max(new), QH, KVH, HD, window, scale,
                         err=err, softcap=cap)
        assert int(err) == 0
    else:
        K.attn_append(ctx, q, k, v, None, starts, pos0, slots, pool, pages, ptab, ring, 3, max(new), QH, KVH, HD, window, scale,
                      tensor_cores=impl == "mma", softcap=cap)
    at = 0
    for s, p, n in zip(seqs, past, new):
        r = s.to(dtype).float()
        ref = capped_attention(r[:, 0, :QH], r[:, 1, :KVH], r[:, 2, :KVH], window, scale, cap, first=p)
        close(ctx[at:at + n].view(n, QH, HD), ref, dtype)
        at += n


# ------------------------------------------------------------------------------------------ taps, rotation, values from keys
def _batch(lengths, starts, slots):
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    tok_seq, tok_pos, seq_start = [], [], [0]
    for b, (n, p) in enumerate(zip(lengths, starts)):
        tok_seq += [b] * n
        tok_pos += list(range(p, p + n))
        seq_start.append(seq_start[-1] + n)
    return types.SimpleNamespace(tok_seq=i32(tok_seq), tok_pos=i32(tok_pos), seq_start=i32(seq_start), seq_pos0=i32(starts),
                                 seq_slot=i32(slots), seq_end=i32([p + n for n, p in zip(lengths, starts)]), B=len(lengths),
                                 T=sum(lengths), max_len=max(lengths))


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 1e-5), (torch.bfloat16, 1.2e-2)])
@pytest.mark.parametrize("H, G, HD, taps, dims, window, cuts", [
    (4, 2, 16, 3, 8, 20, (150,)), (3, 3, 16, 2, 4, 7, (1,) * 30), (2, 1, 24, 5, 24, 70, (33, 2, 65, 1, 1, 1, 40)),
    (2, 1, 64, 4, 32, 0, (64, 64, 3)), (1, 1, 8, 1, 0, 0, (20, 1, 1, 5))])
def test_taps_with_interleaved_rotation_and_values_from_the_keys(K, dtype, tol, H, G, HD, taps, dims, window, cuts):
    """Two sequences through `tap_rotate_store` in steps of the given sizes (whole, single tokens, portions): the step's rows
    [q | turned k | v] and, afterwards, what the ring of pages holds, against the plain filter and rotation."""
    rot = dict(dims=dims, base=300.0, scaling=dict(factor=4.0, original=40, fast=8.0, slow=1.0)) if dims else None
    rate, mag = (None, 1.0)
    if rot:
        r64, mag = plain.rotation(rot)
        rate = r64.to(torch.float32).to(DEV)
    QC, KC = H * HD, G * HD
    g = torch.Generator().manual_seed(taps + HD)
    lengths = [sum(cuts), sum(cuts) - 7]
    proj = [torch.randn(n, QC + KC, generator=g).to(dtype) for n in lengths]
    w = torch.randn(QC + KC, taps, generator=g) * 0.6
    ring = (window + 63) // 64 * 64 if window else 0
    pages_per = max(1, -(-(min(max(lengths), ring) if ring else max(lengths)) // 64))
    pool = torch.full((2, 4 * pages_per, G, 64, HD), float("nan"), dtype=dtype, device=DEV)
    ptab = torch.randperm(4 * pages_per, generator=g).to(torch.int32).view(4, pages_per).to(DEV)
    slots = [2, 1]
    state = torch.zeros(4, taps * (QC + KC), device=DEV) if taps > 1 else None
    want = []
    for n, x in zip(lengths, proj):
        y = plain.taps(x.double(), w.double()) if taps > 1 else x.double() * w.double()[:, 0]
        pos = torch.arange(n)
        qr = plain.turn_pairs(y[:, :QC].view(n, H, HD), pos, rot).reshape(n, QC)
        kr = plain.turn_pairs(y[:, QC:].view(n, G, HD), pos, rot).reshape(n, KC)
        want.append(torch.cat([qr, kr, y[:, QC:]], 1))
    at = [0, 0]
    for cut in cuts:
        lens = [min(cut, n - a) for n, a in zip(lengths, at)]
        live = [i for i in range(2) if lens[i] > 0]
        b = _batch([lens[i] for i in live], [at[i] for i in live], [slots[i] for i in live])
        rows = torch.cat([proj[i][at[i]:at[i] + lens[i]] for i in live]).to(DEV)
        single = all(lens[i] == 1 and at[i] > 0 for i in live)
        out = torch.full((b.T, QC + 2 * KC), float("nan"), dtype=dtype, device=DEV)
        K.tap_rotate_store(rows, None, w.to(DEV), state, out, b, QC, HD, rate, mag, kv=(pool, 4 * pages_per, ptab, G, HD, 0),
                           one_token_each=single, interleaved=True, value_from_key=True, ring=ring, rows_out=True,
                           from_zero=all(at[i] == 0 for i in live))
        ref = torch.cat([want[i][at[i]:at[i] + lens[i]] for i in live])
        assert float((out.double().cpu() - ref).abs().max()) < tol * max(1.0, float(ref.abs().max()))
        for i in live:
            at[i] += lens[i]
    for i, n in enumerate(lengths):                    # the cache: the last `ring` positions (or all), keys turned, values not
        for p in range(max(0, n - ring) if ring else 0, n):
            e = p % ring if ring else p
            page = int(ptab[slots[i], e // 64])
            got = torch.cat([pool[0, page, :, e % 64].reshape(-1), pool[1, page, :, e % 64].reshape(-1)]).double().cpu()
            assert float((got - want[i][p, QC:]).abs().max()) < tol * max(1.0, float(want[i].abs().max())), (i, p)


# ------------------------------------------------------------------------------------------ router and gate
def test_groups_scored_by_their_two_best(K):
    """Corrections and logits are placed so that the group with the single best expert loses to a group whose two best
    sum higher; closed groups count as minus infinity although choice scores are negative; weights come without the
    correction and are renormalised."""
    E, top, W, rows = 8, 3, 16, 40
    g = torch.Generator().manual_seed(3)
    h = torch.randn(rows, W, generator=g)
    router = torch.randn(E, W, generator=g) * 0.8
    correction = torch.tensor([0.9, -2.0, -0.3, -0.2, -1.5, -1.4, 0.1, 0.15])
    P = {"x.router": router.double(), "x.correction": correction.double()}
    for groups, keep, best in [((4, 2), 2, 2), ((4, 3), 3, 2), ((2, 1), 1, 2), ((8, 5), 5, 2), ((4, 2), 2, 1)]:
        ids = torch.empty(rows * top, dtype=torch.int32, device=DEV)
        wts = torch.empty(rows * top, dtype=torch.float32, device=DEV)
        tiles = K.moe_max_tiles(rows * top, E)
        perm = torch.empty(tiles * K.MOE_TILE_SIMT, dtype=torch.int32, device=DEV)
        dest = torch.empty(rows * top, dtype=torch.int32, device=DEV)
        work = torch.empty(K.moe_work_size(rows * top, E), dtype=torch.int32, device=DEV)
        K.moe_route(ids, wts, perm, dest, work, h.to(DEV), router.to(DEV), None, top, renormalize=True,
                    correction=correction.to(DEV), groups=groups[0], keep=keep, renorm_eps=1e-20, group_best=best)
        if best == 2:
            want_ids, want_w = plain.route(h.double(), P, "x.", dict(experts=E, top=top, groups=dict(count=groups[0], keep=keep)))
            assert torch.equal(ids.view(rows, top).cpu().long(), want_ids)
            assert float((wts.view(rows, top).cpu().double() - want_w).abs().max()) < 1e-6
        else:
            first = ids.view(rows, top).cpu().long()
    # the two rules differ on this input: scoring by the best alone keeps other groups open
    two, _ = plain.route(h.double(), P, "x.", dict(experts=E, top=top, groups=dict(count=4, keep=2)))
    assert not torch.equal(first, two)


@pytest.mark.parametrize("dtype, tol", [(torch.float32, 1e-6), (torch.bfloat16, 8e-3)])
def test_clamped_gate_alone(K, dtype, tol):
    g = torch.Generator().manual_seed(8)
    rows, F, limit = 50, 44, 1.3
    gu = (torch.randn(rows, 2 * F, generator=g) * 2).to(dtype)
    out = torch.empty(rows, F, dtype=dtype, device=DEV)
    K.swiglu(out, gu.to(DEV), act=K.ACT_CLAMPED_SWISH, limit=limit)
    a, b = gu[:, :F].double().clamp(max=limit), gu[:, F:].double().clamp(-limit, limit)
    ref = a * torch.sigmoid(1.702 * a) * (b + 1.0)
    assert float((out.double().cpu() - ref).abs().max()) < tol * float(ref.abs().max())
    assert float((gu[:, :F].double() > limit).double().mean()) > 0.1          # the clamp is at work on this input


@pytest.mark.parametrize("kernel, M", [("skinny", 5), ("skinny", 16), ("few_rows", 40), ("few_rows", 128), ("tiled", 300),
                                       ("tiled256", 700), ("grouped", 384)])
def test_clamped_gate_in_the_products_epilogues(K, kernel, M):
    """a = g' sigmoid(1.702 g') (u' + 1) formed where the product [gate; up] leaves its sums: the streaming product, the
    few-rows and the tiled tcgen05 products, and the grouped one with a matrix per row tile."""
    F, Kin, limit = 136, 192, 0.8
    x = rnd(M, Kin, dtype=torch.bfloat16, seed=1)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device=DEV)

    def plain_rows(rows, w):
        gu = rows.double().cpu() @ w.double().cpu().T
        g = gu[:, :F].to(torch.bfloat16).double().clamp(max=limit)
        u = gu[:, F:].to(torch.bfloat16).double().clamp(-limit, limit)
        return g * torch.sigmoid(1.702 * g) * (u + 1.0)

    if kernel == "grouped":
        w = rnd(3, 2 * F, Kin, dtype=torch.bfloat16, scale=0.12, seed=2)
        groups = torch.tensor([2, 0, 1], dtype=torch.int32, device=DEV)
        K.gemm_tc_grouped(out, x, w, groups, swiglu=3, err=err, block_n=128, limit=limit)
        ref = torch.cat([plain_rows(x[128 * t:128 * (t + 1)], w[int(groups[t])]) for t in range(3)])
    else:
        w = rnd(2 * F, Kin, dtype=torch.bfloat16, scale=0.12, seed=2)
        if kernel == "skinny":
            K.gemm_skinny(out, x, w, swiglu=3, limit=limit)
        elif kernel == "few_rows":
            K.gemm_tc_few_rows(out, x, w, swiglu=3, err=err, limit=limit)
        else:
            K.gemm_tc(out, x, w, swiglu=3, err=err, block_n=256 if kernel == "tiled256" else 128, limit=limit)
        ref = plain_rows(x, w)
    assert int(err) == 0
    assert float((out.double().cpu() - ref).abs().max()) < 1.2e-2 * float(ref.abs().max())
    assert float((ref.abs() > 0.5).double().mean()) > 0.05 and float(ref.max()) <= limit * (limit + 1.0) + 1e-9


@pytest.mark.parametrize("dtype, tensor_cores", [("float32", True), ("bfloat16", True), ("bfloat16", False)])
def test_routed_feed_forward_with_clamped_experts_and_a_shared_one(K, dtype, tensor_cores):
    """The routed part with its grouped products (CUDA cores, and the tcgen05 grouped product with the gate behind it)
    plus the expert that every token runs, as the block's sum sees them, against the plain statement."""
    from catena_models_b200.engine.runtime import Runtime
    from catena_models_b200.parts import build_part

    W, F, E, top, rows = 64, 48, 6, 2, 300
    f = dict(kind="moe", expert=dict(ff=F, limit=0.9), router=dict(experts=E, top=top, groups=dict(count=3, keep=2)),
             shared=dict(ff=32, limit=1.4))
    g = torch.Generator().manual_seed(12)
    n = lambda *s: (torch.randn(*s, generator=g) / s[-1] ** 0.5).to(torch.bfloat16)
    P = {"m.router": n(E, W) * 4, "m.correction": (torch.randn(E, generator=g) * 0.2).to(torch.bfloat16)}
    for e in [f"e{j}." for j in range(E)] + ["shared."]:
        ff = 32 if e == "shared." else F
        P.update({f"m.{e}gate": n(ff, W) * 2, f"m.{e}up": n(ff, W) * 2, f"m.{e}down": n(W, ff)})
    rt = Runtime(getattr(torch, dtype), DEV)
    rt.grouped_tensor_cores = tensor_cores
    routed = build_part("feed_forward", "routed_swiglu", prefix="m.", hidden=W, intermediate=F, experts=E, top=top, gate="sigmoid",
                        renormalize=True, weight_on="output", activation="clamped_swish", limit=0.9, correction_name="correction",
                        groups=3, keep=2, group_best=2, renorm_eps=1e-20)
    shared = build_part("feed_forward", "swiglu", prefix="m.shared.", hidden=W, intermediate=32,
                        names={"gate": "gate", "up": "up", "down": "down"}, out_dtype="float32", activation="clamped_swish", limit=1.4)
    both = build_part("feed_forward", "sum", members=[routed, shared])
    dev = {k: v.to(DEV).to(torch.float32 if dtype == "float32" and v.dim() == 2 else v.dtype) for k, v in P.items()}
    both.bind_all(dev, rt)
    x = (torch.randn(rows, W, generator=g)).to(torch.bfloat16)
    batch = types.SimpleNamespace(kind="prefill", tok_seq=torch.zeros(rows, dtype=torch.int32, device=DEV), shared={},
                                  partial_sums_ok=False)
    terms = both.forward(rt, batch, x.to(DEV).to(getattr(torch, dtype)))
    hsum = torch.zeros(rows, W, dtype=torch.float32, device=DEV)
    K.residual_add_norm(hsum, terms)
    P64 = {k: v.double() for k, v in P.items()}
    if dtype == "bfloat16":
        ids = {}
        _, chosen = plain.moe_ff(x.double(), P64, "m.", f, rd=plain.to_bf16)
        ref, _ = plain.moe_ff(x.double(), P64, "m.", f, ids=chosen)
        tol = 2e-2
    else:
        ref, _ = plain.moe_ff(x.double(), P64, "m.", f)
        tol = 2e-5
    assert float((hsum.double().cpu() - ref).abs().max()) < tol * float(ref.abs().max())


# ------------------------------------------------------------------------------------------ latent attention
@pytest.mark.parametrize("dtype, tol", [("float32", 3e-5), ("bfloat16", 3e-2)])
def test_latent_attention_with_a_magnitude_and_a_layer_that_reads_its_latents(K, dtype, tol):
    """Two latent attention parts over one state unit: the first writes entries whose turned part carries the rescaled
    rotation's magnitude, the second has no W_dkv and reads them; whole, then token by token, against the plain statement."""
    from catena_models_b200.cache.cache import KVView
    from catena_models_b200.engine.runtime import Runtime
    from catena_models_b200.parts import build_part

    W, H, D, R, DV, KR, QR, n = 48, 3, 16, 8, 24, 40, 24, 150
    rot = dict(dims=R, base=300.0, scaling=dict(factor=6.0, original=48, fast=16.0, slow=2.0))
    m = dict(heads=H, dim=D, rot_dim=R, vdim=DV, kv_rank=KR, q_rank=QR, scale=0.2, rot=rot)
    g = torch.Generator().manual_seed(21)
    mat = lambda *s: (torch.randn(*s, generator=g) / s[-1] ** 0.5).to(torch.bfloat16)
    P = {}
    for p in ("a.", "b."):
        P.update({p + "dq": mat(QR, W), p + "dq.norm": (1 + 0.1 * torch.randn(QR, generator=g)).to(torch.bfloat16), p + "uq": mat(H * (D + R), QR) * 1.6,
                  p + "uk": mat(H * D, KR), p + "uv": mat(H * DV, KR), p + "g": mat(H, W), p + "o": mat(W, H * DV)})
    P.update({"a.dkv": mat(KR + R, W), "a.dkv.norm": (1 + 0.1 * torch.randn(KR, generator=g)).to(torch.bfloat16)})
    rt = Runtime(getattr(torch, dtype), DEV)
    pos = lambda: build_part("position", "paired_rotary", dims=R, theta=300.0, factor=6.0, original=48, fast=16.0, slow=2.0)
    parts = [build_part("mixer", "latent_attention", prefix=p, hidden=W, heads=H, dim=D, rot_dim=R, value_dim=DV, kv_rank=KR,
                        q_rank=QR, position=pos(), scale=0.2, eps=1e-6, output_gate=True, shares_latents=p == "b.", out_dtype="float32")
             for p in ("a.", "b.")]
    assert parts[0].magnitude == pytest.approx(0.1 * math.log(6.0) + 1.0) and parts[1].state_spec() is None
    dev = {k: v.to(DEV).to(torch.float32 if dtype == "float32" and v.dim() == 2 else v.dtype) for k, v in P.items()}
    for part in parts:
        part.bind_all(dev, rt)
    spec = parts[0].state_spec()
    pool = torch.full((1, 8, 1, 64, spec.head_dim), float("nan"), dtype=rt.dtype, device=DEV)
    ptab = torch.tensor([[0, 0, 0], [5, 2, 7]], dtype=torch.int32, device=DEV)
    xa, xb = torch.randn(n, W, generator=g).to(torch.bfloat16), torch.randn(n, W, generator=g).to(torch.bfloat16)
    P64 = {k: v.double() for k, v in P.items()}
    rd = plain.to_bf16 if dtype == "bfloat16" else plain.ident
    ya, kept = plain.latent_attention(xa.double(), P64, "a.", m, 1e-6, rd=rd)
    yb, _ = plain.latent_attention(xb.double(), P64, "b.", m, 1e-6, lent=kept, rd=rd)

    def step(lo, hi, kind):
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        b = types.SimpleNamespace(kind=kind, prefill=kind == "prefill", append=kind == "append", T=hi - lo, B=1, max_len=hi - lo, max_end=hi,
                                  tok_seq=i32([0] * (hi - lo)), tok_pos=i32(list(range(lo, hi))), seq_start=i32([0, hi - lo]),
                                  seq_pos0=i32([lo]), seq_end=i32([hi]), seq_slot=i32([1]), lengths=[hi - lo], positions=[lo], shared={},
                                  partial_sums_ok=False)
        outs = []
        for part, x, owned in ((parts[0], xa, True), (parts[1], xb, False)):
            view = KVView(spec, pool, 8, ptab, 0, owned=owned, unit=0)
            outs.append(part.forward(rt, b, x[lo:hi].to(DEV).to(rt.dtype), view).double().cpu())
        return outs

    got = [step(0, 100, "prefill")] + [step(t, t + 1, "decode") for t in range(100, 130)] + [step(130, n, "append")]
    for j, ref in enumerate((ya, yb)):
        out = torch.cat([s[j] for s in got])
        assert float((out - ref).abs().max()) < tol * float(ref.abs().max()), j
