"""Pafelorn models end to end through the registry, the engine and its cache: small configurations with random weights, compared with
the plain float64 restatement (tests/pafelorn_oracle.py) of whole sequences.  Sizes are chosen unlike each other on purpose: key and
value sizes that differ, several key groups under differential attention, rotation of a part of a head and of the whole head, head
sizes that are no multiple of four, one recurrent block and several, one convolution tap and several, one expert per token and
several, with and without identity experts / shared expert / bigram table / logit cap, layers without feed-forward, a first layer
of every type, keys and values borrowed from a layer that is not layer 0."""
import copy

import numpy as np
import pytest
import torch

import pafelorn_oracle as O

pytestmark = pytest.mark.gpu


def diff(heads=4, kv_heads=2, dim=8, vdim=12, window=20, rot=4, base=500.0, factor=2.0, scale=0.3, d=0.4, kv_from=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": d, "mask": {"size": window}}
    if rot:
        m["rot"] = {"dims": rot, "base": base, "scaling": {"factor": factor}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def par(heads=6, kv_heads=3, dim=12, vdim=8, window=24, rot=6, base=2000.0, scale=0.25, width=40, ls=0.7, rs=1.2, mlp=None,
        bands=(3.0, 1.0, 4.0, 128)):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}}
    if rot:
        left["rot"] = {"dims": rot, "base": base}
        if bands:
            left["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), bands))
    return {"type": "parallel", "mixer": {"left": left, "right": {"width": width}, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


def par2(heads=4, kv_heads=1, dim=10, vdim=6, window=18, keep=3, cap=5.0, rot=10, base=100.0, factor=1.5, scale=0.3, width=36, blocks=3, conv=3, mlp=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": cap, "mask": {"size": window, "keep_first": keep}}
    if rot:
        left["rot"] = {"dims": rot, "base": base, "scaling": {"factor": factor}}
    return {"type": "parallel_2", "mixer": {"left": left, "right": {"width": width, "blocks": blocks, "conv": conv}}, "mlp": mlp}


def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, identity=2, top=2, ff=12, limit=1.5, shared=20, shared_limit=0.7):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared:
        m["shared"] = {"ff": shared, "limit": shared_limit}
    return m


def config(layers, vocab=61, width=48, eps=1e-5, scale=2.0, bigram=(37, 5, 11), cap=12.0):
    c = {"architecture": "Pafelorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale}, "layers": layers}
    if bigram:
        c["embedding"]["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    if cap:
        c["logit_softcap"] = cap
    return c


CONFIGS = {
    "mixed": config([diff(mlp=dense()), par(mlp=moe()), par2(), diff(heads=2, kv_heads=1, dim=6, vdim=4, window=9, rot=6, factor=3.0, mlp=moe(experts=4, identity=0, top=1, shared=0)),
                     diff(kv_from=0, mlp=moe(experts=3, identity=3, top=3, ff=8, limit=0.9, shared=8, shared_limit=2.0)), par2(heads=2, kv_heads=2, dim=4, vdim=4, window=7, keep=9, rot=2, width=8, blocks=1, conv=1, mlp=dense(20))]),
    "odd": config([par2(heads=3, kv_heads=3, dim=6, vdim=5, window=11, keep=0, cap=2.0, rot=0, width=22, blocks=2, conv=5, mlp=moe(experts=3, identity=1, top=2, ff=10, limit=3.0, shared=6, shared_limit=3.0)),
                   par(heads=2, kv_heads=1, dim=6, vdim=10, window=5, rot=6, bands=None, width=13, ls=1.0, rs=0.25, mlp=None),
                   diff(heads=3, kv_heads=3, dim=10, vdim=7, window=13, rot=0, d=0.1, mlp=dense(30)),
                   diff(heads=3, kv_heads=3, dim=10, vdim=7, window=4, rot=0, d=0.8, kv_from=2, mlp=None)], vocab=33, width=44, eps=1e-3, scale=1.0, bigram=None, cap=0.0),
    "wide": config([par(heads=8, kv_heads=2, dim=64, vdim=80, window=70, rot=32, base=20000.0, width=160, mlp=moe(experts=12, identity=4, top=4, ff=32, limit=2.5, shared=40, shared_limit=1.0)),
                    diff(heads=6, kv_heads=3, dim=32, vdim=48, window=33, rot=16, mlp=dense(160)),
                    par2(heads=4, kv_heads=2, dim=72, vdim=64, window=66, keep=70, cap=30.0, rot=24, width=128, blocks=4, conv=4, mlp=moe(experts=12, identity=0, top=2, ff=32, shared=0))],
                   vocab=130, width=96, bigram=(101, 7, 3)),
}
CONFIGS["long"] = config([par2(heads=4, kv_heads=2, dim=16, vdim=16, window=130, keep=5, cap=25.0, rot=8, width=64, blocks=2, conv=3, mlp=moe(experts=8, identity=2, top=3, ff=24, shared=24)),
                          diff(heads=4, kv_heads=1, dim=16, vdim=24, window=40, rot=16, base=10000.0, mlp=dense(96)),
                          par(heads=4, kv_heads=2, dim=24, vdim=16, window=150, rot=8, base=10000.0, width=48, mlp=moe(experts=8, identity=0, top=2, ff=24, shared=0)),
                          diff(heads=4, kv_heads=1, dim=16, vdim=24, window=70, rot=16, base=10000.0, kv_from=1, mlp=None)], vocab=77, width=64)


# heads as wide as they come in served models: key / value tiles that need the opt-in shared memory sizes
CONFIGS["big"] = config([par(heads=4, kv_heads=2, dim=256, vdim=256, window=80, rot=64, base=50000.0, width=72, mlp=dense(64)),
                         diff(heads=2, kv_heads=1, dim=128, vdim=256, window=50, rot=128, base=50000.0, mlp=None),
                         par2(heads=2, kv_heads=1, dim=96, vdim=160, window=60, keep=2, cap=40.0, rot=96, width=40, blocks=5, conv=2, mlp=moe(experts=2, identity=1, top=1, ff=16, shared=16))],
                        vocab=50, width=128, bigram=(11, 3, 5), cap=0.0)


class Case:
    def __init__(self, name, tmp, dtype):
        from blazr_b200 import registry
        self.cfg = copy.deepcopy(CONFIGS[name])
        self.P = O.random_model(self.cfg, seed=11)
        O.write_checkpoint(str(tmp), self.cfg, self.P)
        self.model = registry.load_model(str(tmp), "cuda:0", dtype)
        self._ref = {}

    def engine(self, **kw):
        from blazr_b200.engine import Engine
        return Engine(self.model, **kw)

    def ref(self, tokens):
        key = tuple(tokens)
        if key not in self._ref:
            self._ref[key] = O.forward(self.cfg, self.P, list(tokens))
        return self._ref[key]


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    made = {}

    def get(name, dtype="float32"):
        if (name, dtype) not in made:
            made[(name, dtype)] = Case(name, tmp_path_factory.mktemp(f"{name}_{dtype}"), dtype)
        return made[(name, dtype)]
    return get


def toks(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def err(got, ref):
    d = torch.as_tensor(got).double() - ref.double()
    d = d - d.mean(-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt() / ref.double().std()).max().item()


def err_rows(got, ref):
    d = torch.as_tensor(got).double() - ref.double()
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / ref.double().std()


TOL32, TOL16 = 5e-5, 6e-2


@pytest.mark.parametrize("name", ["mixed", "odd", "wide", "big"])
def test_whole_prompt_and_layers(cases, name):
    c = cases(name)
    n = 90 if name in ("wide", "big") else 53
    t = toks(n, c.cfg["vocab"], 1)
    eng = c.engine(max_tokens=96, max_seqs=2)
    got = eng.run_entries([{"id": "a", "tokens": t, "want": list(range(n))}], ["a"])
    assert err(got, c.ref(t)) < TOL32
    from blazr_b200.batch import StepEntry, build_step
    seq = eng.cache.admit("b")
    eng.cache.reserve(seq, len(t))
    dbg = []
    c.model.forward(build_step([StepEntry(t, 0, seq.slot, seq.blocks, [0])], eng.cache.block_size), debug_layers=dbg)
    outs = []
    O.forward(c.cfg, c.P, t, layers_out=outs)
    assert len(dbg) == len(outs)
    for g, r in zip(dbg, outs):
        assert (g.double() - r).abs().max().item() < 2e-5 * r.abs().max().item()


@pytest.mark.parametrize("name", ["mixed", "odd", "wide", "long"])
def test_bfloat16_mode_stays_close(cases, name):
    """a portion long enough for the tensor-core paths (plain and gated epilogues, experts over sorted pairs, per-block gate projections), then single tokens"""
    c = cases(name, "bfloat16")
    t = toks(100, c.cfg["vocab"], 2)
    eng = c.engine(max_tokens=112, max_seqs=1)
    got = eng.run_entries([{"id": "a", "tokens": t[:70], "want": list(range(70))}], [])
    rows = [eng.run_entries([{"id": "a", "tokens": [t[i]], "want": [0]}], [])[0] for i in range(70, 100)]
    # Where two expert-choice scores of a token lie closer than the 16-bit rounding of the router's input, the choice may fall the other way and
    # that row is off by an expert's share (by a whole expert where a token has one of few); such rows are few, all others are close
    e = err_rows(np.concatenate([got, np.stack(rows)]), c.ref(t))
    assert e.median().item() < TOL16 / 4 and e.quantile(0.85).item() < TOL16 and e.max().item() < 1.0


@pytest.mark.parametrize("name", ["mixed", "odd", "wide", "big"])
def test_prefill_then_token_by_token(cases, name):
    """long decoding: the decoded tokens cross page borders and leave every window; recurrent state, convolution tail and the previous token
    are carried token by token"""
    c = cases(name)
    n = 100
    t = toks(n, c.cfg["vocab"], 3)
    ref = c.ref(t)
    eng = c.engine(max_tokens=112, max_seqs=1)
    got = [eng.run_entries([{"id": "a", "tokens": t[:9], "want": [0, 8]}], [])]
    assert err(got[0], ref[[0, 8]]) < TOL32
    for i in range(9, n):
        got = eng.run_entries([{"id": "a", "tokens": [t[i]], "want": [0]}], [])
        assert err(got, ref[i:i + 1]) < TOL32, f"decoded position {i}"
    assert eng.cache.live["a"].n_tokens == n


def test_decode_from_the_very_first_token(cases):
    """the first tokens of a sequence: the bigram table's last row, an empty state, zeros in front of the convolution, a soft-max of one key and the sink"""
    for name in ("odd", "mixed"):
        c = cases(name)
        t = toks(14, c.cfg["vocab"], 4)
        ref = c.ref(t)
        eng = c.engine(max_tokens=16, max_seqs=1)
        for i in range(14):
            got = eng.run_entries([{"id": "a", "tokens": [t[i]], "want": [0]}], [])
            assert err(got, ref[i:i + 1]) < TOL32, f"{name}: position {i}"


@pytest.mark.parametrize("name,sizes", [("mixed", [2, 3, 2, 17, 1, 24, 2, 2, 30, 5]), ("wide", [15, 2, 64, 1, 1, 65, 2, 63, 40, 129, 2]), ("odd", [1, 2, 4, 5, 6, 50, 20])])
def test_portions_of_changing_size(cases, name, sizes):
    """portions cut in the middle of pages and of windows, down to two tokens: a portion's first tokens read the carried convolution tail,
    the carried previous token, and keys of earlier portions just inside and just outside their windows"""
    c = cases(name)
    n = sum(sizes)
    t = toks(n, c.cfg["vocab"], 5)
    ref = c.ref(t)
    eng = c.engine(max_tokens=-(-n // 16) * 16, max_seqs=1)
    lo = 0
    for s in sizes:
        got = eng.run_entries([{"id": "a", "tokens": t[lo:lo + s], "want": list(range(s))}], [])
        assert err(got, ref[lo:lo + s]) < TOL32, f"portion at {lo} of {s}"
        lo += s


def test_unequal_requests_in_one_batch_with_reused_pages_and_slots(cases):
    """four live requests at most, a pool far smaller than the sum of all requests: finished requests hand their pages and their state slot
    (recurrent state, convolution tail: left as they were) to new ones while others are in the middle of their prompt or decoding"""
    c = cases("mixed")
    V = c.cfg["vocab"]
    seqs = {n: toks(L, V, 20 + i) for i, (n, L) in enumerate([("a", 70), ("b", 9), ("c", 31), ("d", 2), ("e", 48), ("f", 17), ("g", 1), ("h", 26)])}
    eng = c.engine(max_tokens=176, max_seqs=4)
    plan = [[("a", 30), ("b", 2), ("c", 1)], [("c", 5), ("a", 1), ("b", 7), ("d", 2)], [("a", 25), ("e", 3), ("c", 25)], [("e", 45), ("a", 1), ("f", 2)],
            [("a", 13), ("f", 15), ("g", 1), ("h", 2)], [("h", 1)], [("h", 23)]]
    fed = {n: 0 for n in seqs}
    used_pages, used_slots = {}, {}
    for step in plan:
        entries, end = [], []
        for n, k in step:
            entries.append({"id": n, "tokens": seqs[n][fed[n]:fed[n] + k], "want": list(range(k))})
            if fed[n] + k == len(seqs[n]):
                end.append(n)
        got = eng.run_entries(entries, [])
        for n, _ in step:
            used_pages[n], used_slots[n] = list(eng.cache.live[n].blocks), eng.cache.live[n].slot
        for n in end:
            eng.release(n)
        o = 0
        for n, k in step:
            assert err(got[o:o + k], c.ref(seqs[n])[fed[n]:fed[n] + k]) < TOL32, f"{n} at {fed[n]}"
            o += k
            fed[n] += k
    assert all(fed[n] == len(s) for n, s in seqs.items())
    all_pages = [p for v in used_pages.values() for p in v]
    assert len(all_pages) > len(set(all_pages))                      # pages went through several owners
    assert len(set(used_slots.values())) < len(used_slots)           # so did slots
    assert eng.cache.pages.free_blocks == eng.cache.pages.num_blocks and eng.cache.slots.free_slots == 4


def test_alone_and_in_a_batch_agree(cases):
    c = cases("wide")
    V = c.cfg["vocab"]
    a, b = toks(60, V, 30), toks(21, V, 31)
    alone = c.engine(max_tokens=64, max_seqs=1)
    ra = alone.run_entries([{"id": "a", "tokens": a, "want": [59]}], ["a"])
    both = c.engine(max_tokens=112, max_seqs=2)
    both.run_entries([{"id": "b", "tokens": b[:20], "want": []}], [])
    rb = both.run_entries([{"id": "b", "tokens": b[20:], "want": [0]}, {"id": "a", "tokens": a, "want": [59]}], [])
    assert err(rb[1:2], torch.from_numpy(ra)) < 1e-5
    assert err(rb[0:1], c.ref(b)[20:21]) < TOL32


def test_four_decoding_requests_side_by_side(cases):
    c = cases("wide")
    V = c.cfg["vocab"]
    seqs = [toks(12 + 3 * i, V, 70 + i) for i in range(4)]
    eng = c.engine(max_tokens=128, max_seqs=4)
    eng.run_entries([{"id": str(i), "tokens": s[:-4], "want": []} for i, s in enumerate(seqs)], [])
    for k in range(4, 0, -1):
        got = eng.run_entries([{"id": str(i), "tokens": [s[-k]], "want": [0]} for i, s in enumerate(seqs)], [])
        ref = torch.stack([c.ref(s)[len(s) - k] for s in seqs])
        assert err(got, ref) < TOL32


def test_constants_are_read_from_the_configuration(cases):
    """the same weights under another constant give logits that differ by many times the tolerance: were one of them fixed in code or
    ignored, the comparison above could not have passed for these configurations"""
    c = cases("mixed")
    t = toks(40, c.cfg["vocab"], 6)
    ref = c.ref(t)
    eng = c.engine(max_tokens=48, max_seqs=1)
    assert err(eng.run_entries([{"id": "a", "tokens": t, "want": list(range(40))}], ["a"]), ref) < TOL32

    def changed(edit, P=None):
        w = copy.deepcopy(c.cfg)
        edit(w)
        return err(O.forward(w, P or c.P, t), ref)
    L = lambda w, i: w["layers"][i]["mixer"]
    assert changed(lambda w: w["embedding"].update(scale=2.1)) > 20 * TOL32
    assert changed(lambda w: w["embedding"]["bigram"].update(mul_prev=6)) > 20 * TOL32
    assert changed(lambda w: w["embedding"]["bigram"].update(buckets=36)) > 20 * TOL32
    assert changed(lambda w: w.update(logit_softcap=11.0)) > 20 * TOL32
    assert changed(lambda w: L(w, 0).update(diff=0.45)) > 20 * TOL32
    assert changed(lambda w: L(w, 0)["mask"].update(size=19)) > 20 * TOL32
    assert changed(lambda w: L(w, 0)["rot"]["scaling"].update(factor=2.2)) > 20 * TOL32
    assert changed(lambda w: L(w, 1).update(left_scale=0.75)) > 20 * TOL32
    assert changed(lambda w: L(w, 1).update(right_scale=1.1)) > 20 * TOL32
    assert changed(lambda w: L(w, 1)["left"]["mask"].update(size=23)) > 20 * TOL32
    assert changed(lambda w: L(w, 1)["left"]["rot"]["scaling"].update(high=3.0)) > 20 * TOL32
    assert changed(lambda w: L(w, 1)["left"].update(scale=0.26)) > 20 * TOL32
    assert changed(lambda w: L(w, 2)["left"].update(softcap=4.0)) > 20 * TOL32
    assert changed(lambda w: L(w, 2)["left"]["mask"].update(keep_first=2)) > 20 * TOL32
    assert changed(lambda w: L(w, 2)["left"]["mask"].update(size=17)) > 20 * TOL32
    assert changed(lambda w: w["layers"][1]["mlp"]["expert"].update(limit=1.4)) > 20 * TOL32
    assert changed(lambda w: w["layers"][1]["mlp"]["shared"].update(limit=0.6)) > 20 * TOL32
    assert changed(lambda w: w["layers"][1]["mlp"]["router"].update(top=1)) > 20 * TOL32
    assert changed(lambda w: w["norm"].update(eps=1e-3)) > 20 * TOL32
    for name in ("l1.mix.left.sink", "l1.mix.left.temp", "l1.mlp.correction", "l1.mix.left.o.b", "l1.mix.right.z.b", "l2.mix.right.conv.b", "l2.mix.right.ri.b", "l0.mix.q.b"):
        # (a shift of all corrections alike would leave every choice as it was)
        other = {k: ((-3.0 * v if name.endswith("correction") else v + 0.25) if k == name else v) for k, v in c.P.items()}
        assert changed(lambda w: None, other) > 20 * TOL32, name


def test_greedy_generation_through_the_scheduler(cases):
    from blazr_b200.engine import SamplingParams
    c = cases("mixed")
    V = c.cfg["vocab"]
    prompts = [toks(n, V, 40 + i) for i, n in enumerate([5, 33, 1, 12, 20, 3])]
    eng = c.engine(max_tokens=224, max_seqs=3, max_step_tokens=40, prefill_chunk=16)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=6))
    for p, o in zip(prompts, outs):
        seq = list(p)
        for k in range(6):
            lg = O.forward(c.cfg, c.P, seq)[-1]
            top = torch.topk(lg, 2).values
            if (top[0] - top[1]).item() >= 1e-3 * lg.std().item():      # a near tie may fall either way in 32-bit: follow the engine
                assert int(lg.argmax()) == o[k], f"token {k} of prompt of {len(p)}"
            seq.append(o[k])
    assert eng.cache.pages.free_blocks == eng.cache.pages.num_blocks


def test_trace_replay_command(cases, tmp_path):
    """bin/trace_run as a user starts it: steps on standard input, logits files and 'done' lines out"""
    import json
    import os
    import subprocess
    c = cases("odd")
    folder = str(tmp_path / "m")
    O.write_checkpoint(folder, c.cfg, c.P)
    t = toks(30, c.cfg["vocab"], 7)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": t[:20], "want": [19]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": t[20:29], "want": []}, {"id": "y", "tokens": t[:3], "want": [2]}], "end": ["y"]},
             {"step": 2, "entries": [{"id": "x", "tokens": t[29:], "want": [0]}], "end": ["x"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "out")
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out, "--max-tokens", "64"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ref = c.ref(t)
    V = c.cfg["vocab"]
    g = [np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(1, V) for i in range(3)]
    assert err(g[0], ref[19:20]) < TOL32 and err(g[1], ref[2:3]) < TOL32 and err(g[2], ref[29:30]) < TOL32


def test_generate_command(cases, tmp_path):
    """python -m blazr_b200 generate: the checkpoint's config.json picks the design; greedy tokens follow the restatement"""
    import json
    import os
    import subprocess
    import sys
    c = cases("mixed")
    folder = str(tmp_path / "m")
    O.write_checkpoint(folder, c.cfg, c.P)
    prompts = [toks(9, c.cfg["vocab"], 60), toks(2, c.cfg["vocab"], 61)]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "blazr_b200", "generate", "--model", folder, "--dtype", "float32", "--max-new", "4"]
    for p in prompts:
        cmd += ["--prompt", ",".join(str(t) for t in p)]
    r = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [l["prompt"] for l in lines] == prompts
    for l in lines:
        seq = list(l["prompt"])
        assert len(l["tokens"]) == 4
        for tok in l["tokens"]:
            lg = O.forward(c.cfg, c.P, seq)[-1]
            top = torch.topk(lg, 2).values
            if (top[0] - top[1]).item() >= 1e-3 * lg.std().item():
                assert int(lg.argmax()) == tok
            seq.append(tok)


@pytest.mark.parametrize("dtype,tol", [("float32", TOL32), ("bfloat16", TOL16)])
def test_long_portions_next_to_single_tokens(cases, dtype, tol):
    """portions of hundreds of tokens (query tiles over many key tiles, windows far shorter than the prompt, kept first tokens in tiles of
    their own, experts over sorted pairs) in the same steps as single tokens of another request; then both decode side by side"""
    c = cases("long", dtype)
    a, b = toks(420, c.cfg["vocab"], 20), toks(160, c.cfg["vocab"], 21)
    ra, rb = c.ref(a), c.ref(b)
    eng = c.engine(max_tokens=592, max_seqs=2)
    seen = []

    def check(got, ref, what=""):
        if dtype == "float32":
            assert err(got, ref) < tol, what
        seen.append(err_rows(got, ref))

    check(eng.run_entries([{"id": "b", "tokens": b[:3], "want": [2]}], []), rb[2:3])
    wa = [0, 4, 5, 39, 40, 41, 63, 64, 65, 69, 70, 71, 127, 128, 129, 130, 131, 134, 135, 149, 150, 151, 255, 256, 299]
    got = eng.run_entries([{"id": "a", "tokens": a[:300], "want": wa}, {"id": "b", "tokens": [b[3]], "want": [0]}], [])
    check(got, torch.cat([ra[wa], rb[3:4]]))
    got = eng.run_entries([{"id": "b", "tokens": b[4:135], "want": [0, 130]}, {"id": "a", "tokens": a[300:370], "want": [0, 1, 69]}], [])
    check(got, torch.cat([rb[[4, 134]], ra[[300, 301, 369]]]))
    for i in range(25):
        got = eng.run_entries([{"id": "a", "tokens": [a[370 + i]], "want": [0]}, {"id": "b", "tokens": [b[135 + i]], "want": [0]}], [])
        check(got, torch.cat([ra[370 + i:371 + i], rb[135 + i:136 + i]]), f"decoded token {i}")
    got = eng.run_entries([{"id": "a", "tokens": a[395:420], "want": [24]}], ["a", "b"])
    check(got, ra[419:420])
    e = torch.cat(seen)      # 16-bit mode: a row whose expert choice is a close call may be off by one expert's share; all but a few rows are close
    assert e.median().item() < tol / 4 + 1e-5 and e.quantile(0.9).item() < tol and e.max().item() < 10 * tol
    from blazr_b200 import seqops
    assert seqops.error_flags() == 0
