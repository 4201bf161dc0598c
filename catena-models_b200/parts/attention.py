"""Grouped-query attention mixer with head RMSNorm on q and k, a position encoding, a full or
sliding causal mask and an optional per-head sigmoid gate on the output.

Order of operations (src/lfm3.rs:390-464): one matrix product over the packed rows
[Wq; Wk; Wv; Wgate] (src/lfm3.rs:1159-1262); head norm and rotation of q and k, k and the raw v
written to the cache (src/catena/lfm3.hex:622-781); scores scaled by 1/sqrt(head_dim), keys
hidden when k > p or, with a window W, when k + W <= p (src/catena/lfm3.hex:48-57); softmax and
the value sum in float; context times sigmoid(gate) per head (src/catena/lfm3.hex:25-46);
output projection.

A prompt step attends over the step's own keys and values (every sequence of such a step
starts at position 0); a decode step attends over the cache; an append step (several tokens on
top of started sequences) reads the keys below each sequence's first new position from the cache
and the rest from the step, and writes the step's keys and values to the cache afterwards, so
that a ring still holds what the step's windows reach back to.  All sizes and switches are
constructor parameters; the part knows neither its layer index nor its model.

Further switches, all off by default: `scale` (the factor on q . k instead of 1/sqrt(head_dim)); `sink_name`
(a learned logit per query head that joins the softmax's denominator and has neither key nor value);
`q_temp` = (coef, every), a factor 1 + coef * ln(floor((p + 1) / every) + 1) on the queries at position p;
`value_dim`, the size of a value head when it differs from the size of a query or key head.  The kernels
and the cache work with one head size, so heads of unequal or odd sizes are padded with zero rows of the
projections up to a common multiple of 16 (zero channels change no score and give zero outputs, which meet
zero columns of the output projection); `out_dtype` = "float32" leaves the output projection's result in float.

`softcap` = c > 0 bounds every score before the mask and the softmax: s <- c * tanh(s / c), s = (q . k) * scale.

`taps` = K >= 1 puts a short causal filter behind the query and key projections, one set of K taps per channel
(`q_taps`, `k_taps` name the tensors, [channels, K]): y_t = sum_j w[:, j] u_(t - K + 1 + j), zeros before the sequence's
start, before the rotation (K = 1 is a factor per channel; 0: no filter and no tensors).  For K > 1 the last K projected
rows of a sequence are part of the layer's state (float32, a ring beside the key/value pages).  `value_from_key`: the layer has no value projection; a position's value is its key
as the filter leaves it, before the rotation.  Filter, rotation and the cache write are one kernel
(`kernels.tap_rotate_store`), which leaves the step's rows as [q | turned k | v] for the attention kernels.
"""
from __future__ import annotations


import torch

from .. import kernels
from ..cache.spec import CompositeStateSpec, FixedStateSpec, KVStateSpec
from ..csrc.limits import ATTN_DECODE_CHUNK
from ..weights.loader import TensorSpec
from .base import Mixer, register_part
from .linear import Linear


class GQAttention(Mixer):
    prompt_capturable = True
    fused_decode_ok = True
    supports_append = True

    def __init__(self, prefix, hidden, heads, kv_heads, head_dim, window, position, qk_norm_eps,
                 output_gate, names=None, shares_kv=False, scale=None, sink_name=None, q_temp=None, value_dim=None,
                 out_dtype=None, softcap=0.0, taps=0, value_from_key=False):
        names = names or {}
        n = lambda key, default: prefix + names.get(key, default)
        qk_dim, v_dim = head_dim, value_dim or head_dim
        if v_dim != qk_dim or (scale is not None and qk_dim % 16):
            head_dim = -(-max(qk_dim, v_dim) // 16) * 16       # one padded head size for q, k and v
            if qk_norm_eps is not None and head_dim != qk_dim:
                raise ValueError("a head norm over padded heads is not built")
        pad_qk = (heads, qk_dim, head_dim) if head_dim != qk_dim else None
        pad_k = (kv_heads, qk_dim, head_dim) if head_dim != qk_dim else None
        pad_v = (kv_heads, v_dim, head_dim) if head_dim != v_dim else None
        self.qk_dim, self.v_dim = qk_dim, v_dim
        self.softcap, self.taps, self.value_from_key = float(softcap or 0.0), int(taps or 0), bool(value_from_key)
        if self.softcap < 0.0 or self.taps < 0:
            raise ValueError("GQAttention: softcap >= 0 and taps >= 0")
        if self.value_from_key and (v_dim != qk_dim or shares_kv):
            raise ValueError("GQAttention: values that are the keys have the keys' size, and a layer of its own keys")
        if (self.taps > 0 or self.value_from_key) and (shares_kv or qk_norm_eps is not None or q_temp or output_gate):
            raise ValueError("GQAttention: the filtered form has neither head norm, query temperature, gate nor shared keys")
        self.filtered = self.taps > 0 or self.value_from_key
        if self.filtered:
            self.fused_decode_ok = False       # its decode step runs a kernel of its own between the products
        self.sink_name, self.sink = (prefix + sink_name if sink_name else None), None
        self.q_temp = (float(q_temp[0]), int(q_temp[1])) if q_temp else None
        self.out_dtype = {None: None, "float32": torch.float32}[out_dtype]
        self.hidden, self.heads, self.kv_heads, self.head_dim = hidden, heads, kv_heads, head_dim
        self.window = int(window or 0)
        self.position = position
        self.qk_norm_eps = qk_norm_eps           # None: no head norm
        self.output_gate = bool(output_gate)
        self.q_size, self.kv_size = heads * head_dim, kv_heads * head_dim
        # shares_kv: this layer has no key/value projections of its own; it attends over the keys
        # and values of the layer that owns the state unit the plan gives it
        self.shares_kv = bool(shares_kv)
        mats, rows, pads = [n("q", "attn_q.weight")], [heads * qk_dim], [pad_qk]
        if not self.shares_kv:
            mats.append(n("k", "attn_k.weight"))
            rows.append(kv_heads * qk_dim)
            pads.append(pad_k)
            if not self.value_from_key:
                mats.append(n("v", "attn_v.weight"))
                rows.append(kv_heads * v_dim)
                pads.append(pad_v)
        if self.output_gate:
            mats.append(n("gate", "attn_gate.weight"))
            rows.append(heads)
            pads.append(None)
        self.qkvg = Linear(mats, rows, hidden, head_rows=pads)
        self.out = Linear(n("out", "attn_output.weight"), hidden, heads * v_dim,
                          head_cols=(heads, v_dim, head_dim) if head_dim != v_dim else None)
        self.q_norm_name, self.k_norm_name = n("q_norm", "attn_q_norm.weight"), n("k_norm", "attn_k_norm.weight")
        self.q_norm_w = self.k_norm_w = None
        self.tap_names = (n("q_taps", "attn_q.conv"), n("k_taps", "attn_k.conv")) if self.taps > 0 else ()
        self.tap_w = None
        # 1/sqrt(head_dim) in float32, as the reference bakes it (src/catena/qwen35_wmma_attention.hex:3-22)
        self.scale = float(torch.tensor(1.0, dtype=torch.float32) / torch.sqrt(torch.tensor(float(qk_dim), dtype=torch.float32)))
        if scale is not None:
            self.scale = float(scale)

    def children(self):
        return [self.qkvg, self.out, self.position]

    def tensor_specs(self):
        specs = [TensorSpec(self.sink_name, (self.heads,), "vector")] if self.sink_name else []
        if self.taps > 0:
            specs += [TensorSpec(self.tap_names[0], (self.heads * self.qk_dim, self.taps), "conv"),
                      TensorSpec(self.tap_names[1], (self.kv_heads * self.qk_dim, self.taps), "conv")]
        if self.qk_norm_eps is None:
            return specs
        specs.append(TensorSpec(self.q_norm_name, (self.head_dim,), "norm"))
        if not self.shares_kv:
            specs.append(TensorSpec(self.k_norm_name, (self.head_dim,), "norm"))
        return specs

    def bind(self, tensors, rt):
        self._bound = []
        if self.filtered:
            if self.taps > 0:
                # heads padded with zero channels get taps of zero
                padded = []
                for t in self.tap_names:
                    w = tensors[t].to(torch.float32).view(-1, self.qk_dim, self.taps)
                    full = torch.zeros((w.shape[0], self.head_dim, self.taps), dtype=torch.float32, device=w.device)
                    full[:, :self.qk_dim] = w
                    padded.append(full.view(-1, self.taps))
                self.tap_w = torch.cat(padded).contiguous()
            else:
                self.tap_w = torch.ones((self.q_size + self.kv_size, 1), dtype=torch.float32, device=rt.device)
            self._bound.append(self.tap_w)
        if self.sink_name:
            self.sink = tensors[self.sink_name].to(torch.float32).contiguous()
            self._bound.append(self.sink)
        if self.qk_norm_eps is not None:
            self.q_norm_w = tensors[self.q_norm_name].to(torch.float32).contiguous()
            self._bound.append(self.q_norm_w)
            if not self.shares_kv:
                self.k_norm_w = tensors[self.k_norm_name].to(torch.float32).contiguous()
                self._bound.append(self.k_norm_w)

    def state_spec(self):
        kv = KVStateSpec(self.kv_heads, self.head_dim, self.window)
        if self.taps > 1:
            # a ring of `taps` projected rows [q | k] per sequence, the row of position s in row s % taps
            return CompositeStateSpec((kv, FixedStateSpec((self.taps * (self.q_size + self.kv_size),), "float32")))
        return kv

    def _forward_filtered(self, rt, batch, x, state):
        """q and k behind the taps, v = k before the rotation: one kernel leaves [q | turned k | v] side by side
        and, except in an append step (whose attention reads what is older from the cache first), in the cache."""
        QS, KVS, QH, KVH, HD = self.q_size, self.kv_size, self.heads, self.kv_heads, self.head_dim
        kv, own = state.views if self.taps > 1 else (state, None)
        proj = self.qkvg.apply(rt, x)                                    # [T, QS + KVS]
        decode = batch.kind == "decode"
        # a decode step needs the queries only: its keys and values go straight to the cache
        packed = torch.empty((batch.T, QS if decode else QS + 2 * KVS), dtype=x.dtype, device=x.device)
        rate = self.position.rate_table()
        kernels.tap_rotate_store(proj, None, self.tap_w, None if own is None else own.tensor, packed, batch, QS, HD, rate,
                                 getattr(self.position, "magnitude", 1.0),
                                 kv=(kv.pool, kv.pages, kv.ptab, KVH, HD, 0), one_token_each=decode,
                                 interleaved=self.position.pairing == "interleaved", value_from_key=True, ring=kv.ring,
                                 store=not batch.append, rows_out=not decode, from_zero=batch.prefill)
        q = packed[:, :QS]
        ctx = torch.empty((batch.T, QS), dtype=x.dtype, device=x.device)
        if decode:
            entries = kv.spec.entries(kv.spec.length_class(batch.max_end))
            n_chunks = max(1, -(-entries // ATTN_DECODE_CHUNK))
            part_o, part_ml = rt.scratch_attn_decode(batch.B, QH, HD, n_chunks)
            kernels.attn_decode(ctx, q, None, batch.seq_pos0, batch.seq_slot, kv.pool, kv.pages, kv.ptab, kv.ring,
                                self.window, QH, KVH, HD, n_chunks, self.scale, part_o, part_ml, sink=self.sink,
                                softcap=self.softcap)
        else:
            k, v = packed[:, QS:QS + KVS], packed[:, QS + KVS:]
            if batch.append:
                rt.attention_append(ctx, q, k, v, None, batch, kv, QH, KVH, HD, self.window, self.scale, sink=self.sink,
                                    softcap=self.softcap)
                kernels.kv_store(packed[:, QS:], batch.tok_pos, batch.tok_seq, batch.seq_slot, batch.seq_end, kv.pool,
                                 kv.pages, kv.ptab, kv.ring, KVH, HD)
            else:
                rt.attention_prefill(ctx, q, k, v, None, batch, QH, KVH, HD, self.window, self.scale, sink=self.sink,
                                     softcap=self.softcap)
        return self.out.apply(rt, ctx, out_dtype=self.out_dtype)

    def forward(self, rt, batch, x, state):
        QS, KVS, QH, KVH, HD = self.q_size, self.kv_size, self.heads, self.kv_heads, self.head_dim
        if self.filtered:
            return self._forward_filtered(rt, batch, x, state)
        if self.shares_kv != (not state.owned):
            raise ValueError("a layer that shares keys and values must be given another layer's state unit "
                             "by the plan (owns_state=False), and only such a layer")
        proj = self.qkvg.apply(rt, x)                  # [T, QS + 2 KVS (+ QH)], or [T, QS (+ QH)] when sharing
        interleaved = self.position.pairing == "interleaved"
        if self.shares_kv:
            # q only: head norm and rotation over the q heads, nothing written to the cache
            kernels.qk_prepare(proj, self.q_norm_w, None, self.position.rate_table(), batch.tok_pos, batch.tok_seq,
                               batch.seq_slot, batch.seq_end, None, 0, None, 0, QH, 0, HD, self.qk_norm_eps or 0.0,
                               interleaved=interleaved, q_temp=self.q_temp)
            gate = proj[:, QS:] if self.output_gate else None
        else:
            # an append step keeps the cache as it is until its attention has run
            pool = None if batch.append else state.pool
            kernels.qk_prepare(proj, self.q_norm_w, self.k_norm_w, self.position.rate_table(), batch.tok_pos,
                               batch.tok_seq, batch.seq_slot, batch.seq_end, pool, state.pages, state.ptab,
                               state.ring, QH, KVH, HD, self.qk_norm_eps or 0.0, interleaved=interleaved, q_temp=self.q_temp)
            gate = proj[:, QS + 2 * KVS:] if self.output_gate else None
        q = proj[:, :QS]
        ctx = torch.empty((batch.T, QS), dtype=x.dtype, device=x.device)
        if batch.prefill or batch.append:
            if self.shares_kv and batch.append and state.ring:
                raise NotImplementedError("an append step of a layer that shares the keys and values of a sliding "
                                          "layer: the owner's ring no longer holds what this layer's windows need")
            if self.shares_kv:
                # the owner left this step's keys and values for its readers; bring them beside q so
                # that the attention kernel sees one packed buffer
                k_own, v_own = batch.shared[("kv", state.unit)]
                packed = torch.empty((batch.T, QS + 2 * KVS), dtype=x.dtype, device=x.device)
                packed[:, :QS].copy_(q)
                packed[:, QS:QS + KVS].copy_(k_own)
                packed[:, QS + KVS:].copy_(v_own)
                q, k, v = packed[:, :QS], packed[:, QS:QS + KVS], packed[:, QS + KVS:]
            else:
                k, v = proj[:, QS:QS + KVS], proj[:, QS + KVS:QS + 2 * KVS]
                batch.shared[("kv", state.unit)] = (k, v)
            if batch.append:
                rt.attention_append(ctx, q, k, v, gate, batch, state, QH, KVH, HD, self.window, self.scale, sink=self.sink,
                                    softcap=self.softcap)
                if not self.shares_kv:
                    kernels.kv_store(proj[:, QS:QS + 2 * KVS], batch.tok_pos, batch.tok_seq, batch.seq_slot,
                                     batch.seq_end, state.pool, state.pages, state.ptab, state.ring, KVH, HD)
            else:
                rt.attention_prefill(ctx, q, k, v, gate, batch, QH, KVH, HD, self.window, self.scale, sink=self.sink,
                                     softcap=self.softcap)
        else:
            # launched for the longest sequence that this step's length class allows, so that a
            # recording of the step serves every step of the class
            entries = state.spec.entries(state.spec.length_class(batch.max_end))
            n_chunks = max(1, -(-entries // ATTN_DECODE_CHUNK))
            part_o, part_ml = rt.scratch_attn_decode(batch.B, QH, HD, n_chunks)
            kernels.attn_decode(ctx, q, gate, batch.seq_pos0, batch.seq_slot, state.pool, state.pages, state.ptab,
                                state.ring, self.window, QH, KVH, HD, n_chunks, self.scale, part_o, part_ml, sink=self.sink,
                                softcap=self.softcap)
        return self.out.apply(rt, ctx, out_dtype=self.out_dtype, partial_ok=batch.partial_sums_ok and self.out_dtype is None)


register_part("mixer", "gqa_attention", GQAttention)
