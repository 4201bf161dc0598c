"""The Maferax decoder as parts.

The embedding rows pass an RMS norm with one number as weight.  A layer is a `PostNormBlock` on a float32 stream: the
norm stands behind each sum, x <- norm1(a x + mixer(x)), then x <- norm2(a x + feed_forward(x)) with a =
`postln_alpha`, both sublayers reading the stream itself, all norms with one number as weight.  After every layer
the stream is replaced by a learned average over the depth of the stack: the embedding output and every layer's
result so far, each with a coefficient of the layer's own (`l<i>.dwa`).  The mixer is gated linear attention
(`gated_decay_memory`) or an attention over cached latents (`latent_attention`); the feed-forward a dense gated one
with the tanh form of gelu, a routed one (softmax scores, a correction for the choice only, groups of experts,
identity experts, weights renormalised and scaled, applied to the experts' outputs) or none.  The logits are scaled.

Tensor names: `embed`, `embed.norm`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.dwa`, `l<i>.mix.{q,k,v,g,o,norm,a1,a2,a2.b}` or
`l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o}`, `l<i>.mlp.{gate,up,down}` or
`l<i>.mlp.{router,correction,e<j>.{gate,up,down}}`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.maferax import MaferaxConfig
from ..config.registry import register_architecture
from ..engine.definition import ModelDefinition, PlanEntry
from ..parts import build_part
from ..parts.linear import Linear


def _mixer(cfg, i, layer):
    W, m, p = cfg.width, layer.mixer, f"l{i}.mix."
    if layer.type == "gla":
        if m.rank == 0:
            raise ValueError("the decay network's rank is unknown: give 'mixer.rank', or load the model from its tensors")
        return build_part("mixer", "gated_decay_memory", prefix=p, hidden=W, heads=m.heads, dim=m.dim, value_dim=m.vdim,
                          rank=m.rank, tau=m.tau, eps=cfg.norm_eps, out_dtype="float32")
    position = (build_part("position", "paired_rotary", dims=m.rot_dims, theta=m.rot_base) if m.rot_dims
                else build_part("position", "none"))
    return build_part("mixer", "latent_attention", prefix=p, hidden=W, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim,
                      value_dim=m.vdim, kv_rank=m.kv_rank, q_rank=m.q_rank, position=position, scale=m.scale,
                      eps=cfg.norm_eps, output_gate=True, out_dtype="float32")


def _feed_forward(cfg, i, mlp):
    if mlp is None:
        return None
    p = f"l{i}.mlp."
    if mlp.kind == "dense":
        return build_part("feed_forward", "swiglu", prefix=p, hidden=cfg.width, intermediate=mlp.ff,
                          names={"gate": "gate", "up": "up", "down": "down"}, out_dtype="float32", activation="gelu_tanh")
    return build_part("feed_forward", "routed_swiglu", prefix=p, hidden=cfg.width, intermediate=mlp.ff, experts=mlp.experts,
                      top=mlp.top, gate="softmax", renormalize=True, weight_on="output", activation="silu",
                      correction_name="correction", groups=mlp.groups, keep=mlp.keep, identity=mlp.identity, scale=mlp.scale,
                      renorm_eps=1e-20)


def define(cfg: MaferaxConfig) -> ModelDefinition:
    W = cfg.width
    norm = lambda name: build_part("norm", "scalar_rms", name=name, width=W, eps=cfg.norm_eps)
    blocks, plan = [], []
    for i, layer in enumerate(cfg.layers):
        ff = _feed_forward(cfg, i, layer.mlp)
        blocks.append(build_part("block", "postnorm", mixer=_mixer(cfg, i, layer), feed_forward=ff,
                                 mixer_norm=norm(f"l{i}.norm1"), ffn_norm=norm(f"l{i}.norm2") if ff is not None or layer.norm_alone else None,
                                 residual_scale=cfg.postln_alpha, depth_name=f"l{i}.dwa", depth_index=i))
        plan.append(PlanEntry(block=i, state=i))
    return ModelDefinition(architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=W, embedding_name="embed",
                           blocks=blocks, plan=plan, final_norm=norm("final.norm"), head=Linear("head", cfg.vocab, W),
                           logit_scale=cfg.logit_scale, residual_float32=True, embedding_norm=norm("embed.norm"),
                           depth_entries=len(cfg.layers) + 1)


register_architecture("Maferax", MaferaxConfig, define)
