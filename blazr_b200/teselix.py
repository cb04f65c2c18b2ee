"""Teselix: a decoder-only design of post-norm layers with token shift and gated residuals, whose mixers are retention layers (linear
attention with a fixed decay per head) or latent-attention layers (low-rank query / key-value latents, one shared rotated key part,
a learned sink in the soft-max, a sigmoid gate per head), and whose feed-forward is a mixture of experts chosen by a table indexed
with the token id, plus a shared expert.

This module only reads the design's config.json and maps it onto the generic specs of blazr_b200/layered.py (layout "post"); the
mechanisms and their kernels are shared with any other layer-list design:

    config key                              -> spec
    vocab, width                            -> LayeredConfig.vocab / width (one residual stream, output projection = embedding table)
    norm.eps                                -> eps of every layer norm, rms norm and unit norm
    postln_alpha                            -> LayeredConfig.post_alpha: x <- LN(alpha x + gate * sublayer(x))
    layers[i].type = "retention"            -> RetentionSpec(heads, dim, vdim, decay[heads], rot -> RotarySpec(dims, base, layout "half"))
    layers[i].type = "latent_attention"     -> LatentAttentionSpec(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale,
                                               rot -> RotarySpec(dims, base, yarn = scaling.(factor, original, fast, slow), layout "interleaved"))
    layers[i].weights_of = j                -> LayerSpec.weights_of: the tensors of layer j, a cache / state of its own
    layers[i].mlp = null                    -> no feed-forward sublayer
    layers[i].mlp.kind = "moe"              -> MoeFfSpec(router "table", router.experts, router.top, expert.ff, expert.limit, act "swish_clamp",
                                               shared.ff / shared.limit without a token gate)

What the design fixes is in code: the key scale dim^(-1/2) of retention, the unit norm and silu gate behind it, the pairing of rotated
dimensions (halves in retention, neighbours in latent attention), the sink and the head gates of latent attention, the expert form
min(g, limit) * sigmoid(1.702 g) * (clamp(u, -limit, limit) + 1), the expert weight 1 / top.

Tensor names: embed, final.norm(.b), l<i>.norm1(.b), l<i>.norm2(.b), l<i>.shift, l<i>.rg1(.b), l<i>.rg2(.b),
retention l<i>.mix.{q,k,v,g,o}; latent attention l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,g,o};
l<i>.mlp.table, l<i>.mlp.e<j>.{gate,up,down}, l<i>.mlp.shared.{gate,up,down}.
"""
from __future__ import annotations

from .layered import LatentAttentionSpec, LayeredConfig, LayerSpec, MoeFfSpec, RetentionSpec, RotarySpec

ARCHITECTURE = "Teselix"
EXPERT_ACT = "swish_clamp"
EXPERT_ALPHA = 1.702
EXPERT_UP_SHIFT = 1.0


class ConfigError(ValueError):
    pass


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config: {where} lacks '{key}'")
    return d[key]


def _rotary(rot, where: str, layout: str):
    if rot is None:
        return None
    sc = rot.get("scaling")
    yarn = None
    if sc is not None:
        yarn = tuple(float(_need(sc, k, where + ".rot.scaling")) for k in ("factor", "original", "fast", "slow"))
        if yarn[0] <= 0 or yarn[2] <= 0 or yarn[3] <= 0:
            raise ConfigError(f"config: {where}: rotary scaling constants must be positive")
    spec = RotarySpec(dims=int(_need(rot, "dims", where + ".rot")), base=float(_need(rot, "base", where + ".rot")), yarn=yarn, layout=layout)
    if spec.dims < 2 or spec.dims % 2:
        raise ConfigError(f"config: {where}: rot.dims must be even")
    return spec


def _feed_forward(mlp, where: str):
    if mlp is None:
        return None
    kind = _need(mlp, "kind", where)
    if kind != "moe":
        raise ConfigError(f"config: {where}: unknown feed-forward kind '{kind}'")
    r, ex, shared = _need(mlp, "router", where), _need(mlp, "expert", where), mlp.get("shared")
    spec = MoeFfSpec(experts=int(_need(r, "experts", where + ".router")), top=int(_need(r, "top", where + ".router")), ff=int(_need(ex, "ff", where + ".expert")),
                     act=EXPERT_ACT, router="table", limit=float(_need(ex, "limit", where + ".expert")), alpha=EXPERT_ALPHA, up_shift=EXPERT_UP_SHIFT,
                     shared_ff=int(_need(shared, "ff", where + ".shared")) if shared else 0, shared_gate=False,
                     shared_limit=float(_need(shared, "limit", where + ".shared")) if shared else 0.0)
    if not 1 <= spec.top <= spec.experts:
        raise ConfigError(f"config: {where}: router.top must lie between 1 and router.experts")
    return spec


def _mixer(kind: str, m: dict, where: str):
    heads = int(_need(m, "heads", where))
    if heads < 1:
        raise ConfigError(f"config: {where}: heads must be positive")
    if kind == "retention":
        decay = [float(d) for d in _need(m, "decay", where)]
        if len(decay) != heads:
            raise ConfigError(f"config: {where}: one decay per head expected")
        spec = RetentionSpec(heads=heads, dim=int(_need(m, "dim", where)), vdim=int(_need(m, "vdim", where)), decay=decay, rot=_rotary(m.get("rot"), where, "half"))
        if spec.rot is not None and spec.rot.dims > spec.dim:
            raise ConfigError(f"config: {where}: rot.dims exceeds dim")
        return spec
    if kind == "latent_attention":
        spec = LatentAttentionSpec(heads=heads, dim=int(_need(m, "dim", where)), rot_dim=int(m.get("rot_dim", 0)), vdim=int(_need(m, "vdim", where)),
                                   q_rank=int(_need(m, "q_rank", where)), kv_rank=int(_need(m, "kv_rank", where)), scale=float(_need(m, "scale", where)),
                                   rot=_rotary(m.get("rot"), where, "interleaved"), sink=True, gated=True)
        if (spec.rot is None) != (spec.rot_dim == 0) or (spec.rot is not None and spec.rot.dims != spec.rot_dim):
            raise ConfigError(f"config: {where}: rot.dims must equal rot_dim")
        return spec
    raise ConfigError(f"config: {where}: unknown layer type '{kind}'")


def parse_config(cfg: dict) -> LayeredConfig:
    out = LayeredConfig(name=ARCHITECTURE, vocab=int(_need(cfg, "vocab", "top level")), width=int(_need(cfg, "width", "top level")), streams=1, norm_groups=1,
                        eps=float(_need(_need(cfg, "norm", "top level"), "eps", "norm")), canon_taps=0, embed_scale=1.0, layout="post", tied_head=True,
                        depth_average=False, post_alpha=float(_need(cfg, "postln_alpha", "top level")))
    layers = _need(cfg, "layers", "top level")
    for i, lay in enumerate(layers):
        where = f"layers[{i}]"
        kind = _need(lay, "type", where)
        share = lay.get("weights_of")
        if share is not None:
            share = int(share)
            if not 0 <= share < i or layers[share].get("weights_of") is not None:
                raise ConfigError(f"config: {where}: weights_of must name an earlier layer that has tensors of its own")
        out.layers.append(LayerSpec(kind, _mixer(kind, _need(lay, "mixer", where), where), _feed_forward(lay.get("mlp"), where + ".mlp"), weights_of=share))
    return out
