"""Plain statement of the Maferax decoder, one function per mechanism, in float64 on the CPU.

Nothing here is shared with the library: the tests compare the engine's kernels with these functions.
`P` is {tensor name: float64 tensor}; `cfg` is the dict of config.json.  Notation: h [T, W] rows of one
sequence that starts at position `p0`; a state argument, where given, is what an earlier portion returned.

    rms(x)            x / sqrt(mean(x^2) + eps)
    embedding         rms(E[token]) * g_e                         (g: one number)
    layer             y = g_1 rms(a x + mixer(x));  z = g_2 rms(a y + ff(y))           (a = postln_alpha)
    depth average     the next layer reads sum_j d_i[j] X_j over X_0 (embedding) .. X_(i+1) (layer i's z)
    output            (g_f rms(x)) H^T * logit_scale

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


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def turn_pairs(x, positions, dims, base):
    """Rotation of the leading `dims` channels of x [T, ..., n]: channel 2i against 2i + 1 by the angle
    position * base^(-2i/dims); the other channels stay."""
    out = x.clone()
    half = dims // 2
    rate = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    ang = (positions.to(F64)[:, None] * rate[None, :]).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * torch.cos(ang) - v * torch.sin(ang)
    out[..., 1:dims:2] = v * torch.cos(ang) + u * torch.sin(ang)
    return out


def latent_attention(h, P, p, m, eps, p0=0, state=None, rd=ident):
    """Attention whose keys and values are read out of a small latent row per token.  state: (latents
    [n, kv_rank], turned shared key parts [n, rot_dim]) of the positions before p0.  Returns (y, state)."""
    T = h.shape[0]
    H, D, R, DV, KR = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(p0, p0 + T)
    h = rd(h)
    cq = rd(rms(rd(h @ P[p + "dq"].T), eps) * P[p + "dq.norm"])
    q = rd(cq @ P[p + "uq"].T).view(T, H, D + R)
    q_plain, q_turn = q[..., :D], turn_pairs(q[..., D:], pos, m["rot"]["dims"], m["rot"]["base"])
    low = rd(h @ P[p + "dkv"].T)
    c = rd(rms(low[:, :KR], eps) * P[p + "dkv.norm"])
    kt = rd(turn_pairs(low[:, KR:], pos, m["rot"]["dims"], m["rot"]["base"]))
    if state is not None:
        c, kt = torch.cat([state[0], c]), torch.cat([state[1], kt])
    n = c.shape[0]
    k_plain = (c @ P[p + "uk"].T).view(n, H, D)
    v = (c @ P[p + "uv"].T).view(n, H, DV)
    s = (torch.einsum("thd,nhd->htn", q_plain, k_plain) + torch.einsum("thr,nr->htn", q_turn, kt)) * m["scale"]
    seen = torch.arange(n)[None, :] <= pos[:, None]
    s = s.masked_fill(~seen[None], float("-inf"))
    w = torch.softmax(s, -1)
    o = torch.einsum("htn,nhv->thv", w, v)
    o = o * torch.sigmoid(rd(h @ P[p + "g"].T))[:, :, None]
    return rd(o.reshape(T, H * DV)) @ P[p + "o"].T, (c, kt)


def gla_decay(h, P, p, m):
    """Per token, head and key channel: sigmoid(W_2 (W_1 h) + b)^(1/tau)."""
    z = (h @ P[p + "a1"].T) @ P[p + "a2"].T + P[p + "a2.b"]
    return torch.exp(torch.nn.functional.logsigmoid(z) / m["tau"])


def gla(h, P, p, m, eps, state=None, rd=ident):
    """Linear attention with a decay per key channel: S <- diag(a_t) S + k_t v_t^T, o_t = S^T q_t.  state:
    S [H, D, DV] (zeros at the start).  Returns (y, S)."""
    T = h.shape[0]
    H, D, DV = m["heads"], m["dim"], m["vdim"]
    h = rd(h)
    q = rd(h @ P[p + "q"].T).view(T, H, D) * D ** -0.5
    k = rd(h @ P[p + "k"].T).view(T, H, D)
    v = rd(h @ P[p + "v"].T).view(T, H, DV)
    a = gla_decay(h, P, p, m).view(T, H, D)
    S = torch.zeros(H, D, DV, dtype=F64) if state is None else state.clone()
    o = torch.zeros(T, H, DV, dtype=F64)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps) * P[p + "norm"]
    y = o.reshape(T, H * DV) * silu(rd(h @ P[p + "g"].T))
    return rd(y) @ P[p + "o"].T, S


def dense_ff(h, P, p, rd=ident):
    h = rd(h)
    return rd(gelu_tanh(rd(h @ P[p + "gate"].T)) * rd(h @ P[p + "up"].T)) @ P[p + "down"].T


def route(h, P, p, r):
    """(ids [T, top], weights [T, top]) of a router with softmax scores, a correction that only the choice
    sees, groups of neighbouring experts of which the best `keep` stay open, and a scale on the weights."""
    z = h @ P[p + "router"].T
    s = torch.softmax(z, -1)
    choice = s + P[p + "correction"] if p + "correction" in P else s
    groups = r.get("groups")
    if groups:
        n = choice.shape[-1] // groups["count"]
        best = choice.view(-1, groups["count"], n).max(-1).values
        keep = best.topk(groups["keep"], -1).indices
        open_ = torch.zeros_like(best, dtype=torch.bool).scatter_(1, keep, True)
        choice = choice.masked_fill(~open_[:, :, None].expand(-1, -1, n).reshape(choice.shape), float("-inf"))
    ids = choice.topk(r["top"], -1).indices
    w = s.gather(1, ids)
    return ids, w / (w.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)


def routed_ff(h, P, p, mlp, ids=None, rd=ident):
    """Experts 0 .. experts-1 are small gated feed-forwards (silu); the last `identity` router outputs stand for
    experts that return their input.  `ids`: use this choice of experts instead of the router's own."""
    r = mlp["router"]
    if ids is None:
        ids, _ = route(rd(h), P, p, r)
    s = torch.softmax(rd(h) @ P[p + "router"].T, -1)
    w = s.gather(1, ids)
    w = w / (w.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)
    y = torch.zeros_like(h)
    full, h = h, rd(h)
    for t in range(h.shape[0]):
        for e, we in zip(ids[t].tolist(), w[t]):
            if e >= r["experts"]:
                y[t] += we * full[t]
            else:
                q = f"{p}e{e}."
                y[t] += we * (rd(silu(rd(h[t] @ P[q + "gate"].T)) * rd(h[t] @ P[q + "up"].T)) @ P[q + "down"].T)
    return y


def layer(x, P, i, cfg, p0=0, state=None, ids=None, rd=ident, ids_out=None):
    L = cfg["layers"][i]
    eps, a = cfg["norm"]["eps"], cfg["postln_alpha"]
    if L["type"].startswith("latent_attention"):
        y, state = latent_attention(x, P, f"l{i}.mix.", L["mixer"], eps, p0, state, rd)
    else:
        y, state = gla(x, P, f"l{i}.mix.", L["mixer"], eps, state, rd)
    x = rms(a * x + y, eps) * P[f"l{i}.norm1"]
    mlp = L.get("mlp")
    if mlp is not None and mlp["kind"] == "dense":
        x = rms(a * x + dense_ff(x, P, f"l{i}.mlp.", rd), eps) * P[f"l{i}.norm2"]
    elif mlp is not None:
        if ids is None:
            ids, _ = route(rd(x), P, f"l{i}.mlp.", mlp["router"])
        if ids_out is not None:
            ids_out[i] = ids
        x = rms(a * x + routed_ff(x, P, f"l{i}.mlp.", mlp, ids, rd), eps) * P[f"l{i}.norm2"]
    elif f"l{i}.norm2" in P:
        x = rms(a * x, eps) * P[f"l{i}.norm2"]
    return x, state


def forward(tokens, P, cfg, p0=0, states=None, expert_ids=None, rd=ident, ids_out=None):
    """Logits [T, vocab] of `tokens` at positions p0..; `states`: per layer what an earlier call returned;
    `expert_ids` {layer: ids [T, top]}: the experts to use instead of the routers' own choice; `ids_out` (a dict) takes
    the choice that was used.  Returns (logits, states, the stream after every layer [layers, T, W])."""
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens)
    x = rms(P["embed"][tokens], eps) * P["embed.norm"]
    states = states or [None] * len(cfg["layers"])
    outs, new_states, streams = [x], [], []
    for i in range(len(cfg["layers"])):
        xi, st = layer(x, P, i, cfg, p0, states[i], None if expert_ids is None else expert_ids.get(i), rd, ids_out)
        new_states.append(st)
        outs.append(xi)
        x = sum(P[f"l{i}.dwa"][j] * outs[j] for j in range(i + 2))
        streams.append(x)
    logits = rd(rms(x, eps) * P["final.norm"]) @ P["head"].T * cfg["logit_scale"]
    return logits, new_states, torch.stack(streams)
