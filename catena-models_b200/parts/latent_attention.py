"""Attention whose keys and values are read out of one small latent row per token (multi-head latent attention).

Per token, from the mixer's input h (one product over the packed rows [W_dq; W_dkv; W_g]):

    c_q = rms(W_dq h) * w_q                      the query latent (q_rank channels)
    [c' | r] = W_dkv h ;  c = rms(c') * w_kv     the latent (kv_rank channels); r: rot_dim channels, not normed
    r <- turn(r, position)                       one turned key part that all heads share
    g = W_g h                                    one gate logit per head

and per head, with q = [q_plain (dim) | q_turn (rot_dim)] = W_uq c_q, q_turn turned by the position:

    score(i, j) = (q_plain_i . (W_uk c_j) + q_turn_i . r_j) * scale,   j <= i,   softmax over j
    o_i = (sum_j p_ij W_uv c_j) * sigmoid(g_i)

then the output projection over the concatenated heads.  Only [c | r] is cached: one row of kv_rank + rot_dim
channels per token whatever the number of heads (`KVStateSpec(..., planes=1)`).  The kernels never form the heads'
keys and values: W_uk is moved to the query side (a head's query against the cache is [W_uk^T q_plain | q_turn]) and
W_uv behind the weighted sum over the latents, each a product with one matrix per head (`kernels.head_linear`).
Norms, angles, scores, softmax and the sums over the latents are float32.

The position encoding turns the leading `position.dims` channels of the rot_dim part in interleaved pairs; further
channels of that part pass unchanged.  A position encoding with a `magnitude` has it on every sine and cosine, of the
queries' turned part and of the cached key part alike.

`shares_latents`: the layer has no W_dkv.  It reads the entries [c | r] that another layer of the same latent size and
rotation wrote (the plan hands it that layer's state unit, `owns_state=False`), with its own W_uk, W_uv, queries and
gate; in a whole-prompt step of the expanded form it takes the owner's side-by-side copy of the step's entries from
`StepBatch.shared`.

Every kind of step writes its entries to the cache first.  Portions, single tokens and mixed lengths then read all
keys from there (`kernels.latent_attn`, CUDA cores, float32 sums).  A bfloat16 step of whole prompts has a second form:
the step's entries, kept side by side, are multiplied by [W_uk; W_uv] into keys and values per head (the turned part
copied behind each head's key), heads padded with zeros to the 64 or 128 channels of the tensor-core attention kernels
that the other attentions use (`Runtime.attention_prefill`).  The latents it multiplies are the bfloat16 entries that
the cache holds, so both forms see the same keys up to the rounding of the products.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.spec import KVStateSpec
from ..weights.loader import TensorSpec
from .base import Mixer, register_part
from .linear import Linear


class LatentAttention(Mixer):
    prompt_capturable = True
    supports_append = True

    def __init__(self, prefix, hidden, heads, dim, rot_dim, value_dim, kv_rank, q_rank, position, scale, eps,
                 output_gate=True, out_dtype=None, shares_latents=False):
        if min(heads, dim, value_dim, kv_rank, q_rank) < 1 or rot_dim < 0:
            raise ValueError("LatentAttention: sizes must be positive")
        if getattr(position, "dims", 0) and position.pairing != "interleaved":
            raise ValueError("LatentAttention: the turned part is paired 2i with 2i + 1")
        self.prefix, self.hidden = prefix, hidden
        self.heads, self.dim, self.rot_dim, self.value_dim = heads, dim, rot_dim, value_dim
        self.kv_rank, self.q_rank = kv_rank, q_rank
        self.position, self.scale, self.eps = position, float(scale), float(eps)
        self.output_gate = bool(output_gate)
        self.shares_latents = bool(shares_latents)
        self.magnitude = float(getattr(position, "magnitude", 1.0))
        self.out_dtype = {None: None, "float32": torch.float32}[out_dtype]
        self.entry = kernels.latent_entry_size(kv_rank, rot_dim)
        names, rows = [prefix + "dq"], [q_rank]
        if not self.shares_latents:
            names.append(prefix + "dkv")
            rows.append(kv_rank + rot_dim)
        self.gate_off = sum(rows)                       # where the gate logits begin in the packed product's rows
        if self.output_gate:
            names.append(prefix + "g")
            rows.append(heads)
        self.down = Linear(names, rows, hidden)
        self.up_q = Linear(prefix + "uq", heads * (dim + rot_dim), q_rank)
        self.out = Linear(prefix + "o", hidden, heads * value_dim)
        self.wq_norm = self.wkv_norm = self.w_uk_t = self.w_uv = self.w_kvu = self.rate = None
        # the padded head of the expanded prompt form (0: heads too large for the tensor-core attention kernels)
        need = max(dim + rot_dim, value_dim)
        self.expand_head = 64 if need <= 64 else (128 if need <= 128 else 0)
        # Prompts from this many tokens on take the expanded form.  Measured on B200, one prompt, 16 heads of 64 + 32 and
        # 64 over latents of 256, CUDA-core form against expanded form: EXPAND_TABLE
        self.expand_min_tokens = 64

    def children(self):
        return [self.down, self.up_q, self.out, self.position]

    def tensor_specs(self):
        p = self.prefix
        own = [] if self.shares_latents else [TensorSpec(p + "dkv.norm", (self.kv_rank,), "norm")]
        return [TensorSpec(p + "dq.norm", (self.q_rank,), "norm")] + own + [
                TensorSpec(p + "uk", (self.heads * self.dim, self.kv_rank)),
                TensorSpec(p + "uv", (self.heads * self.value_dim, self.kv_rank))]

    def bind(self, tensors, rt):
        p, H = self.prefix, self.heads
        self.wq_norm = tensors[p + "dq.norm"].to(torch.float32).contiguous()
        self.wkv_norm = None if self.shares_latents else tensors[p + "dkv.norm"].to(torch.float32).contiguous()
        # W_uk^T per head [H, kv_rank, dim]: the query side's product; W_uv per head [H, value_dim, kv_rank]
        self.w_uk_t = tensors[p + "uk"].view(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[p + "uv"].view(H, self.value_dim, self.kv_rank).contiguous()
        # a rate per pair of the turned part; pairs that the position encoding does not cover stay (rate 0)
        rate = torch.zeros(max(1, (self.rot_dim + 1) // 2), dtype=torch.float32, device=self.w_uv.device)
        table = self.position.rate_table()
        if table is not None:
            n = min(table.numel(), self.rot_dim // 2)
            rate[:n] = table[:n]
        self.rate = rate
        # [W_uk; W_uv] as stored, [H dim + H value_dim, kv_rank]: the expanded prompt form's product
        self.w_kvu = torch.cat([tensors[p + "uk"], tensors[p + "uv"]], 0).contiguous()
        self._bound = [t for t in (self.wq_norm, self.wkv_norm, self.w_uk_t, self.w_uv, self.w_kvu) if t is not None]

    def state_spec(self):
        return None if self.shares_latents else KVStateSpec(1, self.entry, 0, planes=1)

    def forward(self, rt, batch, x, state):
        H, D, R, DV, KR, QR = self.heads, self.dim, self.rot_dim, self.value_dim, self.kv_rank, self.q_rank
        T, dev = batch.T, x.device
        owned, unit = getattr(state, "owned", True), getattr(state, "unit", -1)
        if self.shares_latents != (not owned):
            raise ValueError("a layer that shares latents must be given another layer's state unit by the plan "
                             "(owns_state=False), and only such a layer")
        if tuple(state.pool.shape[-2:]) != (kernels.PAGE_TOKENS, self.entry):
            raise ValueError("the state unit's entries are not of this layer's latent size")
        pool, ptab = state.pool, state.ptab
        G0, mag = self.gate_off, self.magnitude
        proj = self.down.apply(rt, x)                                   # [T, QR (+ KR + R) (+ H)]
        cq = torch.empty((T, QR), dtype=x.dtype, device=dev)
        HD = self.expand_head
        expand = (batch.kind == "prefill" and HD > 0 and x.dtype == torch.bfloat16 and rt.tensor_core_prompts
                  and batch.max_len >= self.expand_min_tokens and KR % 8 == 0)
        if expand and self.shares_latents:
            entries = batch.shared.get(("latent_entries", unit))
            expand = entries is not None
        else:
            entries = torch.empty((T, self.entry), dtype=x.dtype, device=dev) if expand else None
            if expand:
                batch.shared[("latent_entries", unit)] = entries      # for the layers that read this one's latents
        kernels.latent_prepare(cq, proj, 0, QR, self.wq_norm, self.wkv_norm, self.rate, pool, ptab, batch, H, D, R, KR, QR,
                               self.eps, entries=None if self.shares_latents else entries, mag=mag,
                               make_entry=not self.shares_latents)
        q = self.up_q.apply(rt, cq)                                      # [T, H (D + R)]
        if expand:
            kvu = rt.linear(entries[:, :KR], self.w_kvu)                 # [T, H D + H DV]
            qkv = torch.empty((T, 3 * H * HD), dtype=x.dtype, device=dev)
            kernels.latent_expand(qkv, q, kvu, entries, self.rate, pool, ptab, batch, H, D, R, DV, KR, HD, mag=mag)
            wide = torch.empty((T, H * HD), dtype=x.dtype, device=dev)
            rt.attention_prefill(wide, qkv[:, :H * HD], qkv[:, H * HD:2 * H * HD], qkv[:, 2 * H * HD:],
                                 proj[:, G0:] if self.output_gate else None, batch, H, H, HD, 0, self.scale)
            if HD == DV:
                ctx = wide
            else:
                ctx = torch.empty((T, H, DV), dtype=x.dtype, device=dev)
                ctx.copy_(wide.view(T, H, HD)[:, :, :DV])
                ctx = ctx.view(T, H * DV)
            return self.out.apply(rt, ctx, out_dtype=self.out_dtype)
        qa = torch.empty((T, H * (KR + R)), dtype=torch.float32, device=dev)
        kernels.head_linear(qa, q, self.w_uk_t, H, D + R, KR + R)
        if R:
            kernels.latent_query_turn(qa, q, self.rate, pool, ptab, batch, H, D, R, KR, mag=mag)
        sums = torch.empty((T, H * KR), dtype=torch.float32, device=dev)
        splits, chunk, parts = 1, 0, None
        # one token per sequence over a bfloat16 cache: the heads are the rows of tensor-core products
        mma = (batch.kind == "decode" and T == batch.B and pool.dtype == torch.bfloat16 and KR <= 512
               and kernels.latent_decode_tensor_cores)
        if batch.kind == "decode":
            # sized by the longest sequence that the step's class of lengths allows, so that a recording serves the class
            keys = state.spec.entries(state.spec.length_class(batch.max_end))
            splits, chunk = kernels.latent_attn_splits(T, H, keys, heads_per_block=16 if mma else 32, kv_rank=KR)
            if splits > 1:
                parts = rt.scratch("latent_attn_parts", T * H * splits * (2 + KR))
        kernels.latent_attn(sums, qa, proj[:, G0:] if self.output_gate else None, pool, ptab, batch, H, R, KR,
                            self.scale, splits=splits, chunk=chunk, parts=parts, tensor_cores=mma)
        ctx = torch.empty((T, H * DV), dtype=x.dtype, device=dev)
        kernels.head_linear(ctx, sums, self.w_uv, H, KR, DV)
        return self.out.apply(rt, ctx, out_dtype=self.out_dtype)


register_part("mixer", "latent_attention", LatentAttention)
