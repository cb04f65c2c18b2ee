"""Host side of the Teselix design (no GPU): the configuration reader and its errors, the registry, the checkpoint writer of the
restatement against the package's safetensors reader."""
import copy

import pytest
import torch

import teselix_oracle as O
from blazr_b200 import registry, teselix
from blazr_b200.layered import LatentAttentionSpec, MoeFfSpec, RetentionSpec, RotarySpec

_RET = {"type": "retention", "mixer": {"heads": 2, "dim": 8, "vdim": 12, "decay": [0.9, 0.99], "rot": {"dims": 4, "base": 77.0}},
        "mlp": {"kind": "moe", "expert": {"ff": 10, "limit": 1.5}, "router": {"experts": 4, "top": 3}, "shared": {"ff": 6, "limit": 0.5}}}
CFG = {"architecture": "Teselix", "vocab": 50, "width": 32, "norm": {"eps": 1e-4}, "postln_alpha": 1.75, "layers": [
    _RET,
    {"type": "latent_attention", "mixer": {"heads": 3, "dim": 6, "rot_dim": 4, "vdim": 5, "q_rank": 7, "kv_rank": 9, "scale": 0.3,
                                           "rot": {"dims": 4, "base": 10.0, "scaling": {"factor": 2.5, "original": 40, "fast": 6.0, "slow": 0.5}}}, "mlp": None},
    dict(copy.deepcopy(_RET), weights_of=0),
    {"type": "latent_attention", "mixer": {"heads": 1, "dim": 6, "rot_dim": 2, "vdim": 5, "q_rank": 7, "kv_rank": 9, "scale": 0.3, "rot": {"dims": 2, "base": 10.0}},
     "mlp": {"kind": "moe", "expert": {"ff": 10, "limit": 2.0}, "router": {"experts": 2, "top": 1}}}]}


def test_config_maps_onto_the_generic_specs():
    c = registry.LAYERED["Teselix"](CFG)
    assert (c.layout, c.tied_head, c.streams, c.canon_taps, c.vocab, c.width, c.eps, c.post_alpha) == ("post", True, 1, 0, 50, 32, 1e-4, 1.75)
    assert c.layers[0].kind == "retention" and c.layers[0].mixer == RetentionSpec(2, 8, 12, [0.9, 0.99], RotarySpec(4, 77.0, None, "half"))
    assert c.layers[0].ff == MoeFfSpec(experts=4, top=3, ff=10, act="swish_clamp", shared_ff=6, shared_gate=False, router="table", limit=1.5, alpha=1.702, up_shift=1.0,
                                       shared_limit=0.5)
    assert c.layers[1].mixer == LatentAttentionSpec(3, 6, 4, 5, 7, 9, 0.3, RotarySpec(4, 10.0, (2.5, 40.0, 6.0, 0.5), "interleaved"), True, True)
    assert c.layers[1].ff is None and c.layers[1].weights_of is None
    assert c.layers[2].weights_of == 0 and c.layers[2].mixer == c.layers[0].mixer and c.layers[2].ff == c.layers[0].ff
    assert c.layers[3].ff.shared_ff == 0 and c.layers[3].ff.top == 1 and c.layers[3].mixer.rot.yarn is None


def _broken(edit):
    c = copy.deepcopy(CFG)
    edit(c)
    return c


@pytest.mark.parametrize("edit", [
    lambda c: c.pop("vocab"), lambda c: c.pop("postln_alpha"), lambda c: c["norm"].pop("eps"), lambda c: c["layers"][0].update(type="mamba2"),
    lambda c: c["layers"][0]["mixer"].update(decay=[0.9]), lambda c: c["layers"][0]["mixer"]["rot"].update(dims=5),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), lambda c: c["layers"][1]["mixer"]["rot"].update(dims=2),
    lambda c: c["layers"][1]["mixer"].pop("kv_rank"), lambda c: c["layers"][1]["mixer"].pop("rot"), lambda c: c["layers"][0]["mlp"].update(kind="dense"),
    lambda c: c["layers"][0]["mlp"]["router"].update(top=5), lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"),
    lambda c: c["layers"][2].update(weights_of=2), lambda c: c["layers"][2].update(weights_of=3), lambda c: c["layers"][3].update(weights_of=2)])
def test_config_errors_are_named(edit):
    with pytest.raises(teselix.ConfigError):
        teselix.parse_config(_broken(edit))


def test_checkpoint_round_trip_and_shared_layers(tmp_path):
    """layers that borrow another layer's tensors add none to the checkpoint; integer tables keep their type"""
    from blazr_b200.safetensors_loader import load_checkpoint
    P = O.random_model(CFG, seed=3)
    assert not any(k.startswith("l2.") for k in P) and "l1.norm2" not in P and "l3.mlp.shared.up" not in P
    O.write_checkpoint(str(tmp_path), CFG, P)
    cfg, st = load_checkpoint(str(tmp_path))
    assert cfg == CFG and registry.architecture_of(str(tmp_path)) == "Teselix"
    assert st.dtype("l0.mlp.table") == "I32" and torch.equal(st.tensor("l0.mlp.table"), P["l0.mlp.table"])
    assert torch.equal(st.tensor("l1.mix.sink").float(), P["l1.mix.sink"])
    rows = P["l0.mlp.table"]
    assert all(len(set(r.tolist())) == 3 for r in rows)
    st.close()


def test_restatement_is_causal_and_carries_the_shift():
    """the restatement itself: a later token changes no earlier logits; the first token sees a zero predecessor"""
    P = O.random_model(CFG, seed=4)
    t = [3, 9, 27, 11, 40, 2]
    full = O.forward(CFG, P, t)
    assert torch.allclose(O.forward(CFG, P, t[:4]), full[:4], atol=1e-12)
    assert not torch.allclose(O.forward(CFG, P, t[1:2]), full[1:2], atol=1e-3)
    x = torch.arange(6.0).view(3, 2)
    assert torch.equal(O.token_shift(x, torch.tensor([1.0, 0.0])), torch.tensor([[0.0, 1.0], [0.0, 3.0], [2.0, 5.0]]))
