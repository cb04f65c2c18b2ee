"""Host side of the Pafelorn design (no GPU): config.json -> generic specs, rotary frequency tables against the plain restatement,
the previous token carried by the cache manager into the step arrays, rejected configurations."""
import copy

import numpy as np
import pytest

import pafelorn_oracle as O
from blazr_b200 import pafelorn, registry
from blazr_b200.batch import StepEntry, build_step
from blazr_b200.cache import CacheManager
from blazr_b200.layered import AttentionSpec, DenseFfSpec, MinGruSpec, MoeFfSpec, RgLruSpec, RotarySpec, TwoBranchSpec


def cfg():
    att = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3, "diff": 0.4, "mask": {"size": 20}, "rot": {"dims": 4, "base": 500.0, "scaling": {"factor": 2.0}}}
    left1 = {"heads": 6, "kv_heads": 3, "dim": 12, "vdim": 8, "scale": 0.25, "mask": {"size": 24},
             "rot": {"dims": 6, "base": 2000.0, "scaling": {"factor": 3.0, "low": 1.0, "high": 4.0, "original": 128}}}
    left2 = {"heads": 4, "kv_heads": 1, "dim": 10, "vdim": 6, "scale": 0.3, "softcap": 5.0, "mask": {"size": 18, "keep_first": 3}, "rot": {"dims": 10, "base": 100.0}}
    moe = {"kind": "moe", "expert": {"ff": 12, "limit": 1.5}, "router": {"experts": 5, "identity": 2, "top": 2}, "shared": {"ff": 20, "limit": 0.7}}
    return {"architecture": "Pafelorn", "vocab": 61, "width": 48, "norm": {"eps": 1e-5}, "logit_softcap": 12.0,
            "embedding": {"scale": 2.0, "bigram": {"buckets": 37, "mul_prev": 5, "mul_cur": 11}},
            "layers": [{"type": "attention", "mixer": att, "mlp": {"kind": "dense", "ff": 56}},
                       {"type": "parallel", "mixer": {"left": left1, "right": {"width": 40}, "left_scale": 0.7, "right_scale": 1.2}, "mlp": moe},
                       {"type": "parallel_2", "mixer": {"left": left2, "right": {"width": 36, "blocks": 3, "conv": 3}}, "mlp": None},
                       {"type": "attention", "mixer": dict(att, kv_from=0), "mlp": None}]}


def test_registered_and_mapped_onto_generic_specs():
    assert registry.LAYERED["Pafelorn"] is pafelorn.parse_config
    c = pafelorn.parse_config(cfg())
    assert (c.layout, c.vocab, c.width, c.tied_head, c.bigram, c.logit_softcap, c.embed_scale) == ("out_norm", 61, 48, False, (37, 5, 11), 12.0, 2.0)
    a, p1, p2, s = c.layers
    assert a.kind == "attention" and isinstance(a.mixer, AttentionSpec) and a.mixer.diff == 0.4 and a.mixer.bias and a.mixer.qk_norm == "head" and a.mixer.window == 20
    assert a.mixer.rot.layout == "half" and a.mixer.rot.linear == 2.0 and a.mixer.rot.bands is None and not a.mixer.gated
    assert isinstance(a.ff, DenseFfSpec) and a.ff.act == "polynorm" and a.ff.ff == 56
    assert p1.kind == "two_branch" and isinstance(p1.mixer, TwoBranchSpec) and isinstance(p1.mixer.right, MinGruSpec) and p1.mixer.right.width == 40
    assert (p1.mixer.left_scale, p1.mixer.right_scale, p1.mixer.branch_norm) == (0.7, 1.2, False)
    L = p1.mixer.left
    assert L.sink and L.head_temp and L.out_bias and L.bias and L.rot.layout == "interleaved" and L.rot.bands == (3.0, 1.0, 4.0, 128.0) and L.rot.linear == 1.0
    f = p1.ff
    assert isinstance(f, MoeFfSpec) and (f.router, f.experts, f.identity, f.top, f.ff, f.limit, f.shared_ff, f.shared_limit, f.correction) == ("softmax", 5, 2, 2, 12, 1.5, 20, 0.7, True)
    assert isinstance(p2.mixer.right, RgLruSpec) and (p2.mixer.right.width, p2.mixer.right.blocks, p2.mixer.right.conv, p2.mixer.right.decay) == (36, 3, 3, 8.0)
    L2 = p2.mixer.left
    assert (L2.qk_norm, L2.softcap, L2.keep_first, L2.window, L2.gated, L2.gate_elem, L2.sink, L2.bias) == ("full", 5.0, 3, 18, True, True, False, False)
    assert p2.mixer.branch_norm and p2.mixer.left_scale == 0.5 and p2.mixer.right_scale == 0.5 and p2.ff is None
    assert s.mixer.kv_from == 0 and s.ff is None


@pytest.mark.parametrize("rot", [{"dims": 8, "base": 250.0}, {"dims": 8, "base": 250.0, "scaling": {"factor": 4.0}},
                                 {"dims": 16, "base": 900.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}},
                                 {"dims": 6, "base": 30.0, "scaling": {"factor": 2.5, "low": 0.5, "high": 3.0, "original": 20}}])
def test_frequency_tables(rot):
    sc = rot.get("scaling") or {}
    banded = "original" in sc
    spec = RotarySpec(dims=rot["dims"], base=rot["base"], linear=1.0 if banded else sc.get("factor", 1.0),
                      bands=(sc["factor"], sc["low"], sc["high"], sc["original"]) if banded else None)
    fr, amp = spec.table()
    assert amp == 1.0
    np.testing.assert_allclose(fr, np.asarray(O.rotary_frequencies(rot)), rtol=1e-6)
    if banded:      # the three bands all occur in these tables
        plain = np.asarray(O.rotary_frequencies({"dims": rot["dims"], "base": rot["base"]}))
        ratio = fr / plain
        assert np.isclose(ratio, 1.0).any() and np.isclose(ratio, 1.0 / sc["factor"]).any() and ((ratio > 1.0 / sc["factor"] + 1e-3) & (ratio < 1.0 - 1e-3)).any()


def test_previous_token_travels_with_the_request():
    cm = CacheManager(64, 2, 16)
    s = cm.admit("a")
    assert s.last_token == -1
    cm.reserve(s, 5)
    sa = build_step([StepEntry([3, 4], 0, s.slot, s.blocks, [1], prev=s.last_token), StepEntry([9], 7, 1, [0], [0], prev=42)], 16)
    assert sa.ent_prev.tolist() == [0, 42] and sa.ent_prev.dtype == np.int32
    assert build_step([StepEntry([1], 0, 0, [0])], 16).ent_prev.tolist() == [0]


@pytest.mark.parametrize("edit,msg", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "exceeds dim"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), "must be even"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=8), "router.top"),
    (lambda c: c["layers"][2]["mixer"]["right"].update(blocks=5), "blocks must divide"),
    (lambda c: c["layers"][1]["mixer"].pop("left_scale"), "lacks 'left_scale'"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"]["scaling"].pop("original"), "lacks 'original'"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "unknown feed-forward kind"),
    (lambda c: c.pop("embedding"), "lacks 'embedding'"),
])
def test_rejected_configurations(edit, msg):
    c = copy.deepcopy(cfg())
    edit(c)
    with pytest.raises(pafelorn.ConfigError, match=msg):
        pafelorn.parse_config(c)


def test_optional_parts_may_be_absent():
    c = cfg()
    del c["embedding"]["bigram"], c["logit_softcap"]
    c["layers"][2]["mixer"]["left"]["mask"].pop("keep_first")
    c["layers"][1]["mlp"].pop("shared")
    c["layers"][1]["mlp"]["router"].pop("identity")
    p = pafelorn.parse_config(c)
    assert p.bigram is None and p.logit_softcap == 0.0 and p.layers[2].mixer.left.keep_first == 0
    assert p.layers[1].ff.shared_ff == 0 and p.layers[1].ff.identity == 0
