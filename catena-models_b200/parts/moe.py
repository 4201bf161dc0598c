"""Routed feed-forward: `experts` small gated feed-forward layers of which every token uses `top`.

Router logits z = W_r h and the scores (sigmoid of each logit, or a softmax over the experts) are float32;
the `top` largest scores are chosen (the lower index among equals) and are the weights, as they are or
divided by their sum (`renormalize`).  `weight_on` says where a weight goes: "input" runs the expert on
weight * h and adds the outputs, "output" runs it on h and adds weight * output.  An expert is
W_down (act(W_gate x) * (W_up x)), act = silu or tanh-gelu.

Routing, the ordering of the (token, choice) pairs by expert and the experts' products all run on the
device from what the router kernel leaves there, so the part launches the same kernels for every step of
a shape and its steps can be recorded.  The result is one float32 row per pair; the block's residual sum
adds a token's rows in the order of its choices.

Further rules of a router, all optional: `correction` (a tensor of one number per router output, added to the scores
for the choice only; the weights are the scores without it); `groups` and `keep` (the router outputs form `groups` equal
groups of neighbours, a group's score is its largest choice score, and only members of the best `keep` groups can be
chosen); `identity` (the last `identity` router outputs stand for experts without matrices whose output is their input
times the weight; they take part in scores, groups and choice like any other); `scale` (a factor on the weights) and
`renorm_eps` (added to the sum that `renormalize` divides by); `group_best` (a group's score is the sum of that many of its
largest choice scores instead of the largest alone).

`activation` "clamped_swish" with `limit` L is an expert of another form: g = min(W_gate x, L), u = clamp(W_up x, -L, L),
a = g sigmoid(1.702 g) (u + 1).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import FeedForward, register_part


class RoutedSwiGLU(FeedForward):
    prompt_capturable = True
    supports_append = True

    def __init__(self, prefix, hidden, intermediate, experts, top, gate="sigmoid", renormalize=False,
                 weight_on="input", activation="silu", expert_name="e{}.", correction_name=None, groups=0, keep=0,
                 identity=0, scale=1.0, renorm_eps=0.0, group_best=1, limit=0.0):
        if gate not in ("sigmoid", "softmax") or weight_on not in ("input", "output") or activation not in kernels.ACTIVATIONS:
            raise ValueError("RoutedSwiGLU: gate sigmoid|softmax, weight_on input|output, activation silu|gelu_tanh|clamped_swish")
        if activation == "clamped_swish" and not limit > 0.0:
            raise ValueError("RoutedSwiGLU: the clamped gate needs its limit")
        if top < 1 or experts < 1:
            raise ValueError(f"RoutedSwiGLU: {top} of {experts} experts")
        self.prefix, self.hidden, self.intermediate = prefix, hidden, intermediate
        self.experts, self.top = experts, top
        self.softmax_gate, self.renormalize = gate == "softmax", bool(renormalize)
        self.weight_on_input, self.gelu = weight_on == "input", activation == "gelu_tanh"
        self.act, self.limit, self.group_best = kernels.ACTIVATIONS[activation], float(limit), int(group_best or 1)
        self.expert_name = expert_name
        self.correction_name, self.groups, self.keep = correction_name, int(groups or 0), int(keep or 0)
        self.identity, self.scale, self.renorm_eps = int(identity or 0), float(scale), float(renorm_eps)
        self.outputs = experts + self.identity                 # what the router scores
        if self.groups and (self.outputs % self.groups or not 1 <= self.keep <= self.groups
                            or self.keep * (self.outputs // self.groups) < top):
            raise ValueError(f"RoutedSwiGLU: {self.groups} groups over {self.outputs} router outputs of which {self.keep} stay open, top {top}")
        if top > self.outputs:
            raise ValueError(f"RoutedSwiGLU: {top} of {self.outputs} router outputs")
        if self.identity and self.weight_on_input:
            raise ValueError("RoutedSwiGLU: identity experts need the weight on the output")
        self.correction = None

    def _names(self, e):
        q = self.prefix + self.expert_name.format(e)
        return q + "gate", q + "up", q + "down"

    def tensor_specs(self):
        H, F = self.hidden, self.intermediate
        specs = [TensorSpec(self.prefix + "router", (self.outputs, H))]
        if self.correction_name:
            specs.append(TensorSpec(self.prefix + self.correction_name, (self.outputs,), "vector"))
        for e in range(self.experts):
            g, u, d = self._names(e)
            specs += [TensorSpec(g, (F, H)), TensorSpec(u, (F, H)), TensorSpec(d, (H, F))]
        return specs

    def bind(self, tensors, rt):
        names = [self._names(e) for e in range(self.experts)]
        self.router = tensors[self.prefix + "router"].contiguous()
        # [E, 2 F, H]: an expert's gate rows, then its up rows; [E, H, F]
        self.w_up = torch.stack([torch.cat([tensors[g], tensors[u]], 0) for g, u, _ in names]).contiguous()
        self.w_down = torch.stack([tensors[d] for _, _, d in names]).contiguous()
        if self.router.dtype != self.w_up.dtype:
            self.router = self.router.to(self.w_up.dtype)
        self._bound = [self.router]
        if self.correction_name:
            self.correction = tensors[self.prefix + self.correction_name].to(torch.float32).contiguous()

    def weight_bytes(self):
        # a step reads the router and, of the experts, what its tokens choose: at most every expert once
        per_expert = (self.w_up[0].numel() + self.w_down[0].numel()) * self.w_up.element_size()
        return self.router.numel() * self.router.element_size() + self.experts * per_expert

    def forward(self, rt, batch, x):
        T, top, E = x.shape[0], self.top, self.experts          # E: experts with matrices (they alone get rows)
        P = T * top
        dev = x.device
        if x.dtype != self.w_up.dtype:
            raise ValueError("RoutedSwiGLU: activations and expert matrices must share a dtype")
        # bfloat16 with rows that TMA can fetch: the grouped tcgen05 product over row tiles of 128; else the CUDA cores
        tensor_cores = (x.dtype == torch.bfloat16 and not self.gelu and self.hidden % 8 == 0 and self.intermediate % 8 == 0
                        and (rt.tensor_core_prompts or batch.kind == "decode")
                        and rt.grouped_tensor_cores)
        tile = kernels.MOE_TILE_TC if tensor_cores else kernels.MOE_TILE_SIMT
        max_tiles = kernels.moe_max_tiles(P, E, tile)
        rows = max_tiles * tile
        ids = torch.empty(P, dtype=torch.int32, device=dev)
        wts = torch.empty(P, dtype=torch.float32, device=dev)
        perm = torch.empty(rows, dtype=torch.int32, device=dev)
        dest = torch.empty(P, dtype=torch.int32, device=dev)
        work = torch.empty(kernels.moe_work_size(P, E, tile), dtype=torch.int32, device=dev)
        xs = torch.empty((rows, self.hidden), dtype=x.dtype, device=dev) if tensor_cores else None
        kernels.moe_route(ids, wts, perm, dest, work, x, self.router, batch.tok_seq, top, self.softmax_gate, self.renormalize, tile,
                          xs=xs, apply_weight=self.weight_on_input, correction=self.correction, groups=self.groups,
                          keep=self.keep, identity=self.identity, scale=self.scale, renorm_eps=self.renorm_eps,
                          group_best=self.group_best)
        a = torch.empty((rows, self.intermediate), dtype=x.dtype, device=dev)
        y = torch.empty((rows, self.hidden), dtype=torch.float32, device=dev)
        if tensor_cores:
            groups = kernels.moe_tile_group(work, P, E, tile)
            kernels.gemm_tc_grouped(a, xs, self.w_up, groups, swiglu=3 if self.act == kernels.ACT_CLAMPED_SWISH else True,
                                    err=rt.error_flag, limit=self.limit,
                                    block_n=rt._tile_width(rows, 2 * self.intermediate, widths=(256, 128)))
            kernels.gemm_tc_grouped(y, a, self.w_down, groups, err=rt.error_flag, block_n=128)
        else:
            kernels.moe_grouped(a, x, self.w_up, work, perm, wts, top, max_tiles, up=True,
                                apply_weight=self.weight_on_input, act=self.act, limit=self.limit)
            kernels.moe_grouped(y, a, self.w_down, work, perm, wts, top, max_tiles, up=False,
                                apply_weight=not self.weight_on_input)
        # the grouped tensor-core product has no weights of its own: on the outputs they ride on the residual sum's pieces
        out = kernels.Terms([(y, 1.0, top, dest, wts) if tensor_cores and not self.weight_on_input else (y, 1.0, top, dest)])
        if self.identity:
            # the identity experts' share: the input itself, from the float32 stream when the block left it for this
            src = batch.shared.get("ff_input_f32")
            src = x if src is None or src.shape != x.shape else src
            same = torch.empty((T, self.hidden), dtype=torch.float32, device=dev)
            kernels.moe_identity(same, src, ids, wts, top, E)
            out.append((same, 1.0, 1))
        return out


register_part("feed_forward", "routed_swiglu", RoutedSwiGLU)
