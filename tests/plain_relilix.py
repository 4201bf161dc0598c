"""Plain statement of the Relilix decoder, one function per mechanism, in float64 on the CPU.

Nothing here is shared with the library: the tests compare the engine's kernels with these functions.  `P` is
{tensor name: float64 tensor}; `cfg` is the dict of config.json; h [T, W] are the rows of one sequence from position 0.

    rms(x)            x / sqrt(mean(x^2) + eps)
    embedding         E[token] * s_e
    layer             x <- x + mixer(w_1 rms(x));  x <- x + ff(w_2 rms(x))
    output            (w_f rms(x)) H^T

`rd` (default: nothing) is applied wherever an engine that keeps activations in bfloat16 would round: the stream as the
products read it, the products' results, the cached rows.  With `to_bf16` the functions give the yardstick for what the
storage format alone costs.
"""
import math

import torch

F64 = torch.float64


def ident(x):
    return x


def to_bf16(x):
    return x.to(torch.bfloat16).to(x.dtype)


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def rotation(rot):
    """(rate per pair, factor on sine and cosine) of a rotation section {dims, base, scaling?}."""
    d, base = rot["dims"], rot["base"]
    rate = [base ** (-2.0 * i / d) for i in range(d // 2)]
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        where = lambda t: d * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo, hi = max(math.floor(where(sc["fast"])), 0), min(math.ceil(where(sc["slow"])), d - 1)
        for i in range(d // 2):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            rate[i] = rate[i] / sc["factor"] * ramp + rate[i] * (1.0 - ramp)
        mag = 0.1 * math.log(sc["factor"]) + 1.0
    return torch.tensor(rate, dtype=F64), mag


def turn_pairs(x, positions, rot):
    """Rotation of the leading rot.dims channels of x [T, ..., n]: channel 2i against 2i + 1 by the angle position *
    rate_i, sine and cosine times the rotation's magnitude; the other channels stay."""
    if not rot:
        return x
    out = x.clone()
    d = rot["dims"]
    rate, mag = rotation(rot)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [d // 2]
    ang = (positions.to(F64)[:, None] * rate[None, :]).reshape(shape)
    c, s = torch.cos(ang) * mag, torch.sin(ang) * mag
    u, v = x[..., 0:d:2], x[..., 1:d:2]
    out[..., 0:d:2] = u * c - v * s
    out[..., 1:d:2] = v * c + u * s
    return out


def taps(u, w):
    """y_t = sum_j w[:, j] u_(t - K + 1 + j) per channel, zeros before the first row.  u [T, C], w [C, K]."""
    T, K = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(K):
            s = t - K + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def window_attention(h, P, p, m, rd=ident):
    """Grouped-query attention behind taps on q and k; the values are the keys before the rotation; capped scores; a
    sliding window."""
    T = h.shape[0]
    H, G, D = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    pos = torch.arange(T)
    q, k = rd(h @ P[p + "q"].T), rd(h @ P[p + "k"].T)
    if m.get("conv"):
        q, k = taps(q, P[p + "q.conv"]), taps(k, P[p + "k.conv"])
    q, k = q.view(T, H, D), k.view(T, G, D)
    v = rd(k)
    q, k = rd(turn_pairs(q, pos, m.get("rot"))), rd(turn_pairs(k, pos, m.get("rot")))
    cap, size = m.get("softcap") or 0.0, (m.get("mask") or {}).get("size", 0)
    out = torch.zeros(T, H, D, dtype=F64)
    for i in range(T):
        first = max(0, i - size + 1) if size else 0
        for hh in range(H):
            g = hh // (H // G)
            s = (k[first:i + 1, g] @ q[i, hh]) * m["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            out[i, hh] = torch.softmax(s, 0) @ v[first:i + 1, g]
    return rd(out.reshape(T, H * D)) @ P[p + "o"].T


def latents(h, P, p, m, eps, rd=ident):
    """What a latent layer caches per token: (normed latent [T, kv_rank], turned shared key part [T, rot_dim])."""
    KR = m["kv_rank"]
    pos = torch.arange(h.shape[0])
    ckv = rd(h @ P[p + "dkv"].T)
    c = rms(ckv[:, :KR], eps) * P[p + "dkv.norm"]
    r = turn_pairs(ckv[:, None, KR:], pos, m.get("rot"))[:, 0]
    return rd(c), rd(r)


def latent_attention(h, P, p, m, eps, lent=None, rd=ident):
    """Attention whose keys and values of all heads are read out of (latent, turned key part) per token; `lent`: those
    of the layer that `kv_from` names.  Returns (y, (latents, key parts))."""
    T = h.shape[0]
    H, D, R, DV = m["heads"], m["dim"], m.get("rot_dim", 0), m.get("vdim", m["dim"])
    pos = torch.arange(T)
    cq = rd(rms(rd(h @ P[p + "dq"].T), eps) * P[p + "dq.norm"])
    q = rd(cq @ P[p + "uq"].T).view(T, H, D + R)
    q_plain, q_turn = q[..., :D], turn_pairs(q[..., D:], pos, m.get("rot"))
    c, r = lent if lent is not None else latents(h, P, p, m, eps, rd)
    k_plain = (c @ P[p + "uk"].T).view(T, H, D)
    v = (c @ P[p + "uv"].T).view(T, H, DV)
    gate = torch.sigmoid(rd(h @ P[p + "g"].T))
    out = torch.zeros(T, H, DV, dtype=F64)
    for i in range(T):
        for hh in range(H):
            s = (k_plain[:i + 1, hh] @ q_plain[i, hh] + r[:i + 1] @ q_turn[i, hh]) * m["scale"]
            out[i, hh] = (torch.softmax(s, 0) @ v[:i + 1, hh]) * gate[i, hh]
    return rd(out.reshape(T, H * DV)) @ P[p + "o"].T, (c, r)


def dense_ff(h, P, p, rd=ident):
    return rd(silu(rd(h @ P[p + "gate"].T)) * rd(h @ P[p + "up"].T)) @ P[p + "down"].T


def clamped_expert(h, P, p, limit, rd=ident):
    g = torch.clamp(rd(h @ P[p + "gate"].T), max=limit)
    u = torch.clamp(rd(h @ P[p + "up"].T), -limit, limit)
    return rd(g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ P[p + "down"].T


def route(h, P, p, r):
    """(chosen experts [T, top], their weights [T, top]) of the router section r."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ P[p + "router"].T)
    choice = s + P[p + "correction"]
    gr = r.get("groups")
    if gr:
        n = E // gr["count"]
        for t in range(h.shape[0]):
            ch = choice[t].clone()
            score = [float(torch.sort(ch[g * n:(g + 1) * n], descending=True).values[:2].sum()) for g in range(gr["count"])]
            order = sorted(range(gr["count"]), key=lambda g: (-score[g], g))
            for g in order[gr["keep"]:]:
                ch[g * n:(g + 1) * n] = -math.inf
            choice[t] = ch
    ids = torch.zeros(h.shape[0], top, dtype=torch.long)
    for t in range(h.shape[0]):
        ch = choice[t].clone()
        for j in range(top):
            best = int(torch.argmax(ch))              # the lowest index among equals
            ids[t, j] = best
            ch[best] = -math.inf
    wts = s.gather(1, ids)
    return ids, wts / (wts.sum(-1, keepdim=True) + 1e-20)


def moe_ff(h, P, p, f, rd=ident, ids=None):
    """ids: the experts to use instead of the router's choice (weights still from this input's scores)."""
    own, wts = route(h, P, p, f["router"])
    if ids is not None:
        s = torch.sigmoid(h @ P[p + "router"].T).gather(1, ids)
        wts = s / (s.sum(-1, keepdim=True) + 1e-20)
    else:
        ids = own
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            out[t] += wts[t, j] * clamped_expert(h[t:t + 1], P, f"{p}e{int(ids[t, j])}.", f["expert"]["limit"], rd)[0]
    if f.get("shared"):
        out = out + clamped_expert(h, P, p + "shared.", f["shared"]["limit"], rd)
    return out, ids


def forward(tokens, P, cfg, rd=ident, expert_ids=None, ids_out=None, streams=None):
    """Logits [T, vocab] of one sequence (in a tuple, as the other plain statements return them).  expert_ids: {layer:
    ids} to pin every router's choice; ids_out: a dict that receives the choices made; streams: a list that receives the
    stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = P["embed"][torch.tensor(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h = rd(rms(x, eps) * P[p + "norm1"])
        if L["type"] == "attention":
            y = window_attention(h, P, p + "mix.", m, rd)
        else:
            lender = m.get("kv_from")
            y, kept[i] = latent_attention(h, P, p + "mix.", m, eps, None if lender is None else kept[lender], rd)
        x = x + y
        f = L.get("mlp")
        if f is not None:
            h = rd(rms(x, eps) * P[p + "norm2"])
            if f["kind"] == "dense":
                x = x + dense_ff(h, P, p + "mlp.", rd)
            else:
                y, ids = moe_ff(h, P, p + "mlp.", f, rd, None if expert_ids is None else expert_ids[i])
                if ids_out is not None:
                    ids_out[i] = ids
                x = x + y
        if streams is not None:
            streams.append(x.clone())
    return ((rd(rms(x, eps) * P["final.norm"])) @ P["head"].T,)
