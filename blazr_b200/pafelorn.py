"""Pafelorn: a decoder-only design whose layers put the RMS norm on the sublayer's output (x <- x + norm(sublayer(x)), the sublayers read x
itself).  Its mixers are differential attention (two soft-max maps per head over the same values, optionally over the keys and values of
an earlier layer's cache) or two branches side by side: a windowed attention (learned sink and temperature per head, or soft-capped scores,
kept first tokens and an element-wise output gate) beside an element-wise gated recurrence (minGRU, or a real-gated linear recurrent unit
behind a short convolution).  The feed-forward is dense with the PolyNorm activation or a mixture of experts with a soft-max router, a
correction that enters the choice only, identity experts and a gated shared expert.  A hashed bigram table joins the embedding; the logits
pass a soft cap.

This module only reads the design's config.json and maps it onto the generic specs of blazr_b200/layered.py (layout "out_norm"); the
mechanisms and their kernels are shared with any other layer-list design:

    config key                              -> spec
    vocab, width                            -> LayeredConfig.vocab / width (one residual stream, own output projection "head")
    norm.eps                                -> eps of every RMS norm (layer, branch, q / k, PolyNorm, differential heads)
    embedding.scale, embedding.bigram       -> embed_scale, bigram = (buckets, mul_prev, mul_cur)
    logit_softcap                           -> LayeredConfig.logit_softcap
    layers[i].type = "attention"            -> AttentionSpec(diff, biases on q / k / v, per-head weighted q / k norm, window = mask.size,
                                               rot layout "half" with linear scaling, kv_from)
    layers[i].type = "parallel"             -> TwoBranchSpec(left = AttentionSpec(biases, output bias, per-head q / k norm, sink, head temperature,
                                               window, rot "interleaved" with band scaling), right = MinGruSpec(width), left_scale, right_scale)
    layers[i].type = "parallel_2"           -> TwoBranchSpec(left = AttentionSpec(q / k norm over the whole projection, softcap, window + keep_first,
                                               element-wise output gate, rot "interleaved" with linear scaling),
                                               right = RgLruSpec(width, blocks, conv), scales 1/2, branch_norm)
    layers[i].mlp = null                    -> no feed-forward sublayer
    layers[i].mlp.kind = "dense"            -> DenseFfSpec(ff, act "polynorm")
    layers[i].mlp.kind = "moe"              -> MoeFfSpec(router "softmax" with correction, router.experts / top / identity, expert.ff / limit,
                                               act "swish_clamp", shared.ff / limit with a sigmoid token gate)

What the design fixes is in code: which options each layer type switches on, the decay constant 8 of the recurrent unit, the expert form
min(g, limit) * sigmoid(1.702 g) * (clamp(u, -limit, limit) + 1), the halves of the second two-branch form.

Tensor names: embed, bigram, head, final.norm, l<i>.norm1, l<i>.norm2; attention l<i>.mix.{q,k,v}(.b), q.norm, k.norm, lq1, lk1, lq2, lk2, o;
two-branch l<i>.mix.left.{q,k,v,o}(.b), q.norm, k.norm, temp, sink, g, out and l<i>.mix.right.{z,x,g,o,y,conv,ra,ri,lam}(.b), out;
l<i>.mlp.{up,down,act}; l<i>.mlp.router, correction, e<j>.{gate,up,down}, shared.{gate,up,down,sg}.
"""
from __future__ import annotations

from .layered import AttentionSpec, DenseFfSpec, LayeredConfig, LayerSpec, MinGruSpec, MoeFfSpec, RgLruSpec, RotarySpec, TwoBranchSpec

ARCHITECTURE = "Pafelorn"
EXPERT_ACT = "swish_clamp"
EXPERT_ALPHA = 1.702
EXPERT_UP_SHIFT = 1.0
LRU_DECAY = 8.0


class ConfigError(ValueError):
    pass


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config: {where} lacks '{key}'")
    return d[key]


def _rotary(rot, where: str, layout: str):
    """scaling with `original`: short wavelengths stay, long ones are divided by the factor, a blend between (low / high name the band);
    scaling with a factor alone: every frequency is divided by it"""
    if rot is None:
        return None
    sc = rot.get("scaling")
    linear, bands = 1.0, None
    if sc is not None:
        factor = float(_need(sc, "factor", where + ".rot.scaling"))
        if factor <= 0:
            raise ConfigError(f"config: {where}: rot.scaling.factor must be positive")
        if "original" in sc or "low" in sc or "high" in sc:
            bands = (factor,) + tuple(float(_need(sc, k, where + ".rot.scaling")) for k in ("low", "high", "original"))
            if bands[2] == bands[1] or bands[1] <= 0 or bands[2] <= 0 or bands[3] <= 0:
                raise ConfigError(f"config: {where}: rot.scaling low / high / original must be positive, low != high")
        else:
            linear = factor
    spec = RotarySpec(dims=int(_need(rot, "dims", where + ".rot")), base=float(_need(rot, "base", where + ".rot")), layout=layout, linear=linear, bands=bands)
    if spec.dims < 2 or spec.dims % 2:
        raise ConfigError(f"config: {where}: rot.dims must be even")
    return spec


def _attention(m, where: str, kind: str) -> AttentionSpec:
    mask = m.get("mask") or {}
    base = dict(heads=int(_need(m, "heads", where)), kv_heads=int(_need(m, "kv_heads", where)), dim=int(_need(m, "dim", where)), vdim=int(_need(m, "vdim", where)),
                scale=float(_need(m, "scale", where)), chunk=0, window=int(mask.get("size", 0)), qk_unit_norm=False)
    if kind == "attention":
        kv_from = m.get("kv_from")
        spec = AttentionSpec(**base, gated=False, rot=_rotary(m.get("rot"), where, "half"), qk_norm="head", bias=True, diff=float(_need(m, "diff", where)),
                             kv_from=int(kv_from) if kv_from is not None else None)
    elif kind == "parallel":
        spec = AttentionSpec(**base, gated=False, rot=_rotary(m.get("rot"), where, "interleaved"), qk_norm="head", bias=True, out_bias=True, head_temp=True, sink=True)
    else:
        spec = AttentionSpec(**base, gated=True, gate_elem=True, rot=_rotary(m.get("rot"), where, "interleaved"), qk_norm="full",
                             softcap=float(m.get("softcap", 0.0)), keep_first=int(mask.get("keep_first", 0)))
    if spec.heads < 1 or spec.kv_heads < 1 or spec.heads % spec.kv_heads:
        raise ConfigError(f"config: {where}: heads is not a multiple of kv_heads")
    if spec.rot is not None and spec.rot.dims > spec.dim:
        raise ConfigError(f"config: {where}: rot.dims exceeds dim")
    if spec.window < 0 or spec.keep_first < 0 or spec.softcap < 0:
        raise ConfigError(f"config: {where}: mask sizes and softcap must not be negative")
    return spec


def _feed_forward(mlp, where: str):
    if mlp is None:
        return None
    kind = _need(mlp, "kind", where)
    if kind == "dense":
        return DenseFfSpec(ff=int(_need(mlp, "ff", where)), act="polynorm")
    if kind == "moe":
        r, ex, shared = _need(mlp, "router", where), _need(mlp, "expert", where), mlp.get("shared")
        spec = MoeFfSpec(experts=int(_need(r, "experts", where + ".router")), top=int(_need(r, "top", where + ".router")), ff=int(_need(ex, "ff", where + ".expert")),
                         act=EXPERT_ACT, router="softmax", identity=int(r.get("identity", 0)), correction=True, limit=float(_need(ex, "limit", where + ".expert")),
                         alpha=EXPERT_ALPHA, up_shift=EXPERT_UP_SHIFT, shared_ff=int(_need(shared, "ff", where + ".shared")) if shared else 0, shared_gate=True,
                         shared_limit=float(_need(shared, "limit", where + ".shared")) if shared else 0.0)
        if spec.experts < 1 or spec.identity < 0 or not 1 <= spec.top <= spec.experts + spec.identity:
            raise ConfigError(f"config: {where}: router.top must lie between 1 and router.experts + router.identity")
        return spec
    raise ConfigError(f"config: {where}: unknown feed-forward kind '{kind}'")


def parse_config(cfg: dict) -> LayeredConfig:
    emb = _need(cfg, "embedding", "top level")
    bg = emb.get("bigram")
    out = LayeredConfig(name=ARCHITECTURE, vocab=int(_need(cfg, "vocab", "top level")), width=int(_need(cfg, "width", "top level")), streams=1, norm_groups=1,
                        eps=float(_need(_need(cfg, "norm", "top level"), "eps", "norm")), canon_taps=0, embed_scale=float(_need(emb, "scale", "embedding")), layout="out_norm",
                        tied_head=False, depth_average=False,
                        bigram=(int(_need(bg, "buckets", "embedding.bigram")), int(_need(bg, "mul_prev", "embedding.bigram")), int(_need(bg, "mul_cur", "embedding.bigram"))) if bg else None,
                        logit_softcap=float(cfg.get("logit_softcap") or 0.0))
    layers = _need(cfg, "layers", "top level")
    for i, lay in enumerate(layers):
        where = f"layers[{i}]"
        kind, m = _need(lay, "type", where), _need(lay, "mixer", where)
        if kind == "attention":
            mixer, spec_kind = _attention(m, where, kind), "attention"
            j = mixer.kv_from
            if j is not None and not (0 <= j < i and layers[j].get("type") == "attention" and layers[j]["mixer"].get("kv_from") is None):
                raise ConfigError(f"config: {where}: kv_from must name an earlier attention layer that has keys and values of its own")
        elif kind in ("parallel", "parallel_2"):
            left = _attention(_need(m, "left", where), where + ".left", kind)
            r = _need(m, "right", where)
            if kind == "parallel":
                mixer = TwoBranchSpec(left, MinGruSpec(width=int(_need(r, "width", where + ".right"))), left_scale=float(_need(m, "left_scale", where)),
                                      right_scale=float(_need(m, "right_scale", where)), branch_norm=False)
            else:
                right = RgLruSpec(width=int(_need(r, "width", where + ".right")), blocks=int(_need(r, "blocks", where + ".right")), conv=int(_need(r, "conv", where + ".right")),
                                  decay=LRU_DECAY)
                if right.blocks < 1 or right.width % right.blocks or not 1 <= right.conv <= 8:
                    raise ConfigError(f"config: {where}: blocks must divide the recurrent width; 1 to 8 convolution taps")
                mixer = TwoBranchSpec(left, right, left_scale=0.5, right_scale=0.5, branch_norm=True)
            spec_kind = "two_branch"
        else:
            raise ConfigError(f"config: {where}: unknown layer type '{kind}'")
        out.layers.append(LayerSpec(spec_kind, mixer, _feed_forward(lay.get("mlp"), where + ".mlp")))
    return out
