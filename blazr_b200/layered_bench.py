"""Throughput of a layer-list design at sizes that resemble a real model's layers (random weights), beside the framework's
dense-attention decoder (blazr_b200/decode.py, Q8_0 weights) of the same width, head layout, feed-forward size and layer count:

    prefill  : one prompt of S tokens as one engine step (tokens/s)
    decode   : B live requests with `ctx` tokens each, one token per request per step (tokens/s; CUDA-graph replay)
    kernels  : every operator of one prefill step and one decode step timed alone (CUDA events around each launch), with its
               algorithmic bytes / FLOPs and the fraction of the roofline it reaches; the like kernels of the decoder beside them

`python bench.py --layered fenorax|gemosun|teselix|pafelorn [--layered-sizes w1024,w2048]` prints the result as one JSON line; bench.py's default
workload and JSON line are untouched.  For Gemosun (parallel attention / feed-forward layers, three of four feed-forwards a mixture of
experts) the closest existing model, Fenorax at the same sizes, runs beside it as well; for Teselix (retention and latent-attention mixers,
table-routed experts) both run beside it: Gemosun is the closest in attention and experts, Fenorax in the recurrence.  For Pafelorn (windowed
attention beside element-wise recurrences, differential attention, soft-max-routed gated experts) Gemosun (windowed attention with rotation,
routed experts) and Fenorax (a recurrence with carried state and a short convolution) run beside it as well.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List

import numpy as np
import torch

from . import seqops
from .engine import Engine
from .layered import LayeredModel

# sizes of one layer group; the layer list is [ssm, attention + ff, ssm, attention + ff]
SIZES: Dict[str, dict] = {
    "w1024": dict(width=1024, heads=16, kv_heads=4, dim=64, ff=4096, ssm_heads=32, ssm_vdim=64, state=64, ssm_groups=2, chunk=1024, vocab=32000),
    "w2048": dict(width=2048, heads=32, kv_heads=8, dim=64, ff=8192, ssm_heads=64, ssm_vdim=64, state=128, ssm_groups=8, chunk=2048, vocab=32000),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=14336, ssm_heads=128, ssm_vdim=64, state=128, ssm_groups=8, chunk=2048, vocab=32000),
}
F32_FMA_TFLOPS_NOMINAL = 148 * 128 * 2 * 1.965e9 / 1e12    # CUDA-core f32 rate at the maximum SM clock (not measured)


def fenorax_config(sz: dict, streams: int = 2, taps: int = 3) -> dict:
    ssm = {"type": "mamba2", "mlp": None,
           "mixer": {"conv": 4, "groups": sz["ssm_groups"], "heads": sz["ssm_heads"], "norm_groups": sz["ssm_groups"], "state": sz["state"], "vdim": sz["ssm_vdim"]}}
    att = {"type": "attention", "mlp": {"kind": "dense", "ff": sz["ff"], "limit": 7.0},
           "mixer": {"dim": sz["dim"], "vdim": sz["dim"], "heads": sz["heads"], "kv_heads": sz["kv_heads"], "scale": sz["dim"] ** -0.5, "mask": {"size": sz["chunk"]}}}
    return {"architecture": "Fenorax", "vocab": sz["vocab"], "width": sz["width"], "streams": streams, "norm": {"eps": 1e-5, "groups": 2}, "canon": {"taps": taps},
            "embedding": {"scale": float(sz["width"]) ** 0.5}, "layers": [ssm, att, ssm, att]}


def gemosun_config(sz: dict, experts: int = 32, top: int = 4) -> dict:
    """four parallel layers of the size's width and head layout: sliding window of `chunk` positions with pooled blocks of 16, rotation of
    half of every head with scaled frequencies; feed-forwards [dense, experts, experts, experts], an expert a quarter of the dense size"""
    def att(mlp):
        return {"type": "attention", "mlp": mlp,
                "mixer": {"dim": sz["dim"], "vdim": sz["dim"], "heads": sz["heads"], "kv_heads": sz["kv_heads"], "scale": sz["dim"] ** -0.5,
                          "mask": {"size": sz["chunk"], "pool": 16},
                          "rot": {"dims": sz["dim"] // 2, "base": 10000.0, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    eff = sz["ff"] // 4
    moe = {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": experts, "top": top, "groups": {"count": 4, "keep": 2}}, "shared": {"ff": eff}}
    return {"architecture": "Gemosun", "vocab": sz["vocab"], "width": sz["width"], "norm": {"eps": 1e-5},
            "layers": [att({"kind": "dense", "ff": sz["ff"]}), att(dict(moe)), att(dict(moe)), att(dict(moe))]}


def teselix_config(sz: dict, experts: int = 32, top: int = 4, kv_rank: int = 256) -> dict:
    """four post-norm layers [retention, latent attention] x 2 of the size's width and head layout, every one with table-routed experts (an
    expert a quarter of the dense size, `top` per token) and a shared expert; retention heads of the size's head size with decays spread
    between 1 - 2^-5 and 1 - 2^-12; latent attention with a key / value latent of `kv_rank`, a query latent of 3/8 of the width and a rotated
    part of half a head"""
    H, D, W = sz["heads"], sz["dim"], sz["width"]
    eff = sz["ff"] // 4
    moe = {"kind": "moe", "expert": {"ff": eff, "limit": 7.0}, "router": {"experts": experts, "top": top}, "shared": {"ff": eff, "limit": 7.0}}
    ret = {"type": "retention", "mlp": dict(moe),
           "mixer": {"heads": H, "dim": D, "vdim": D, "decay": [1.0 - 2.0 ** (-5.0 - 7.0 * h / max(H - 1, 1)) for h in range(H)], "rot": {"dims": D, "base": 1e6}}}
    lat = {"type": "latent_attention", "mlp": dict(moe),
           "mixer": {"heads": H, "dim": D, "rot_dim": D // 2, "vdim": D, "q_rank": 3 * W // 8, "kv_rank": kv_rank, "scale": (D + D // 2) ** -0.5,
                     "rot": {"dims": D // 2, "base": 10000.0, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    return {"architecture": "Teselix", "vocab": sz["vocab"], "width": W, "norm": {"eps": 1e-5}, "postln_alpha": 2.0, "layers": [ret, lat, dict(ret), dict(lat)]}


def pafelorn_config(sz: dict, experts: int = 32, identity: int = 2, top: int = 4) -> dict:
    """four out-norm layers [differential attention + dense, attention | minGRU + experts, attention | gated LRU + dense, differential attention over
    layer 0's keys and values + experts] of the size's width and head layout; windows of `chunk` positions; differential heads are half as many with
    values twice as wide; both recurrences are as wide as the model; an expert is a quarter of the dense size"""
    H, G, D, W = sz["heads"], sz["kv_heads"], sz["dim"], sz["width"]
    eff = sz["ff"] // 4
    moe = {"kind": "moe", "expert": {"ff": eff, "limit": 7.0}, "router": {"experts": experts, "identity": identity, "top": top}, "shared": {"ff": eff, "limit": 7.0}}
    dense = {"kind": "dense", "ff": sz["ff"]}
    diff = {"heads": H // 2, "kv_heads": max(G // 2, 1), "dim": D, "vdim": 2 * D, "scale": D ** -0.5, "diff": 0.2, "mask": {"size": sz["chunk"]},
            "rot": {"dims": D, "base": 500000.0, "scaling": {"factor": 6.0}}}
    left1 = {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "mask": {"size": sz["chunk"]},
             "rot": {"dims": D // 2, "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    left2 = {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "softcap": 30.0, "mask": {"size": sz["chunk"], "keep_first": 4},
             "rot": {"dims": D // 2, "base": 10000.0, "scaling": {"factor": 2.0}}}
    return {"architecture": "Pafelorn", "vocab": sz["vocab"], "width": W, "norm": {"eps": 1e-5}, "logit_softcap": 30.0,
            "embedding": {"scale": float(W) ** 0.5, "bigram": {"buckets": 16381, "mul_prev": 36313, "mul_cur": 27191}},
            "layers": [{"type": "attention", "mixer": diff, "mlp": dense},
                       {"type": "parallel", "mixer": {"left": left1, "right": {"width": W}, "left_scale": 1.0, "right_scale": 1.0}, "mlp": moe},
                       {"type": "parallel_2", "mixer": {"left": left2, "right": {"width": W, "blocks": 8, "conv": 4}}, "mlp": dict(dense)},
                       {"type": "attention", "mixer": dict(diff, kv_from=0), "mlp": dict(moe)}]}


def random_tensors_pafelorn(cfg: dict, device, seed: int = 7):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]

    def rnd(*shape, scale=1.0):
        return (torch.randn(shape, generator=g, device=device) * scale).to(torch.bfloat16)

    ones = lambda *n: torch.ones(*n, dtype=torch.bfloat16, device=device)
    zeros = lambda *n: torch.zeros(*n, dtype=torch.bfloat16, device=device)
    t = {"embed": rnd(V, W, scale=W ** -0.5), "bigram": rnd(cfg["embedding"]["bigram"]["buckets"] + 1, W), "head": rnd(V, W, scale=W ** -0.5), "final.norm": ones(W)}

    def lin(name, o, i, bias=False):
        t[name] = rnd(o, i, scale=i ** -0.5)
        if bias:
            t[name + ".b"] = rnd(o, scale=0.1)

    for i, lay in enumerate(cfg["layers"]):
        p, m, mlp = f"l{i}.", lay["mixer"], lay["mlp"]
        t[p + "norm1"], t[p + "norm2"] = ones(W), ones(W)
        kind = lay["type"]
        a, ap = (m, p + "mix.") if kind == "attention" else (m["left"], p + "mix.left.")
        H, G, D, Vd = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        maps = 2 if kind == "attention" else 1
        b = kind != "parallel_2"
        lin(ap + "q", H * maps * D, W, b)
        if a.get("kv_from") is None:
            lin(ap + "k", G * maps * D, W, b)
            lin(ap + "v", G * Vd, W, b)
            t[ap + "k.norm"] = ones(G * D) if kind == "parallel_2" else ones(D)
        t[ap + "q.norm"] = ones(H * D) if kind == "parallel_2" else ones(D)
        lin(ap + "o", W, H * Vd, kind == "parallel")
        if kind == "attention":
            for nm in ("lq1", "lk1", "lq2", "lk2"):
                t[ap + nm] = rnd(D, scale=0.1)
        elif kind == "parallel":
            t[ap + "temp"], t[ap + "sink"] = ones(H), zeros(H)
            r, C = p + "mix.right.", m["right"]["width"]
            lin(r + "z", C, W, True), lin(r + "x", C, W, True), lin(r + "g", C, W), lin(r + "o", W, C)
        else:
            lin(ap + "g", H * Vd, W)
            r, C, nb, taps = p + "mix.right.", m["right"]["width"], m["right"]["blocks"], m["right"]["conv"]
            lin(r + "y", C, W, True), lin(r + "x", C, W, True), lin(r + "o", W, C)
            t[r + "conv"], t[r + "conv.b"] = rnd(C, taps, scale=0.5), zeros(C)
            for nm in ("ra", "ri"):
                t[r + nm], t[r + nm + ".b"] = rnd(nb, C // nb, C // nb, scale=(C // nb) ** -0.5), zeros(nb, C // nb)
            t[r + "lam"] = rnd(C) - 2.0
            t[p + "mix.left.out"], t[p + "mix.right.out"] = ones(W), ones(W)
        if mlp["kind"] == "dense":
            lin(p + "mlp.up", mlp["ff"], W), lin(p + "mlp.down", W, mlp["ff"])
            t[p + "mlp.act"] = torch.tensor([0.5, 0.3, 0.2, 0.0], device=device).to(torch.bfloat16)
        else:
            rt = mlp["router"]
            lin(p + "mlp.router", rt["experts"] + rt["identity"], W)
            t[p + "mlp.correction"] = zeros(rt["experts"] + rt["identity"])
            for e in range(rt["experts"]):
                lin(p + f"mlp.e{e}.gate", mlp["expert"]["ff"], W), lin(p + f"mlp.e{e}.up", mlp["expert"]["ff"], W), lin(p + f"mlp.e{e}.down", W, mlp["expert"]["ff"])
            lin(p + "mlp.shared.gate", mlp["shared"]["ff"], W), lin(p + "mlp.shared.up", mlp["shared"]["ff"], W), lin(p + "mlp.shared.down", W, mlp["shared"]["ff"])
            lin(p + "mlp.shared.sg", 1, W)
    return lambda name: t[name].cpu()


def random_tensors_teselix(cfg: dict, device, seed: int = 7):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]

    def rnd(*shape, scale=1.0):
        return (torch.randn(shape, generator=g, device=device) * scale).to(torch.bfloat16)

    ones = lambda n: torch.ones(n, dtype=torch.bfloat16, device=device)
    zeros = lambda n: torch.zeros(n, dtype=torch.bfloat16, device=device)
    t = {"embed": rnd(V, W), "final.norm": ones(W), "final.norm.b": zeros(W)}
    for i, lay in enumerate(cfg["layers"]):
        p, m, mlp = f"l{i}.", lay["mixer"], lay["mlp"]
        H = m["heads"]
        for q in ("1", "2"):
            t[p + "norm" + q], t[p + "norm" + q + ".b"] = ones(W), zeros(W)
            t[p + "rg" + q], t[p + "rg" + q + ".b"] = rnd(W, W, scale=W ** -0.5), zeros(W)
        t[p + "shift"] = torch.full((W,), 0.5, dtype=torch.bfloat16, device=device)
        if lay["type"] == "retention":
            D, Vd = m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"] = rnd(H * D, W, scale=W ** -0.5), rnd(H * D, W, scale=W ** -0.5)
            t[p + "mix.v"], t[p + "mix.g"], t[p + "mix.o"] = rnd(H * Vd, W, scale=W ** -0.5), rnd(H * Vd, W, scale=W ** -0.5), rnd(W, H * Vd, scale=(H * Vd) ** -0.5)
        else:
            D, Rd, Vd, R, Rq = m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            t[p + "mix.dq"], t[p + "mix.dq.norm"], t[p + "mix.uq"] = rnd(Rq, W, scale=W ** -0.5), ones(Rq), rnd(H * (D + Rd), Rq, scale=Rq ** -0.5)
            t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = rnd(R + Rd, W, scale=W ** -0.5), ones(R)
            t[p + "mix.uk"], t[p + "mix.uv"] = rnd(H * D, R, scale=R ** -0.5), rnd(H * Vd, R, scale=R ** -0.5)
            t[p + "mix.sink"], t[p + "mix.g"], t[p + "mix.o"] = zeros(H), rnd(H, W, scale=W ** -0.5), rnd(W, H * Vd, scale=(H * Vd) ** -0.5)
        E, top, ff, sf = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"], mlp["shared"]["ff"]
        for e in range(E):
            t[p + f"mlp.e{e}.gate"], t[p + f"mlp.e{e}.up"], t[p + f"mlp.e{e}.down"] = rnd(ff, W, scale=W ** -0.5), rnd(ff, W, scale=W ** -0.5), rnd(W, ff, scale=ff ** -0.5)
        t[p + "mlp.shared.gate"], t[p + "mlp.shared.up"], t[p + "mlp.shared.down"] = rnd(sf, W, scale=W ** -0.5), rnd(sf, W, scale=W ** -0.5), rnd(W, sf, scale=sf ** -0.5)
        # every row names `top` different experts: a random start and a stride that is coprime to the expert count
        start = torch.randint(0, E, (V, 1), generator=g, device=device)
        t[p + "mlp.table"] = ((start + torch.arange(top, device=device)[None, :] * (E // top if E % top == 0 else 1)) % E).to(torch.int32)
    return t.__getitem__


def random_tensors_gemosun(cfg: dict, device, seed: int = 7):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    W = cfg["width"]

    def rnd(*shape, scale=1.0):
        return (torch.randn(shape, generator=g, device=device) * scale).to(torch.bfloat16)

    ones = lambda n: torch.ones(n, dtype=torch.bfloat16, device=device)
    t = {"embed": rnd(cfg["vocab"], W), "head": rnd(cfg["vocab"], W, scale=W ** -0.5), "final.norm": ones(W)}
    for i, lay in enumerate(cfg["layers"]):
        p, m, mlp = f"l{i}.", lay["mixer"], lay["mlp"]
        H, G, D = m["heads"], m["kv_heads"], m["dim"]
        t[p + "norm1"], t[p + "norm2"] = ones(W), ones(W)
        t[p + "mix.q"], t[p + "mix.k"] = rnd(H * D, W, scale=W ** -0.5), rnd(G * D, W, scale=W ** -0.5)
        t[p + "mix.g"], t[p + "mix.o"] = rnd(H, W, scale=W ** -0.5), rnd(W, H * D, scale=(H * D) ** -0.5)
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = rnd(ff, W, scale=W ** -0.5), rnd(ff, W, scale=W ** -0.5), rnd(W, ff, scale=ff ** -0.5)
        else:
            E, ff, sf = mlp["router"]["experts"], mlp["expert"]["ff"], mlp["shared"]["ff"]
            t[p + "mlp.router"] = rnd(E, W, scale=2.0 * W ** -0.5)
            for e in range(E):
                t[p + f"mlp.e{e}.up"], t[p + f"mlp.e{e}.down"] = rnd(ff, W, scale=W ** -0.5), rnd(W, ff, scale=ff ** -0.5)
            t[p + "mlp.shared.up"], t[p + "mlp.shared.down"], t[p + "mlp.shared.sg"] = rnd(sf, W, scale=W ** -0.5), rnd(W, sf, scale=sf ** -0.5), rnd(1, W, scale=W ** -0.5)
        d = torch.full((i + 2,), 0.1 / (i + 1), device=device)
        d[i + 1] = 0.9
        t[p + "dwa"] = d.to(torch.bfloat16)
    return t.__getitem__


def random_tensors(cfg: dict, device, seed: int = 7):
    """name -> tensor function with random weights of the design's shapes, generated on the device"""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    W, S, taps = cfg["width"], cfg["streams"], cfg["canon"]["taps"]

    def rnd(*shape, scale=1.0, dtype=torch.bfloat16):
        return (torch.randn(shape, generator=g, device=device) * scale).to(dtype)

    t = {"embed": rnd(cfg["vocab"], W, scale=W ** -0.5), "final.norm": torch.ones(W, dtype=torch.bfloat16, device=device)}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        for q in ((1, 2) if lay["mlp"] else (1,)):
            t[f"{p}norm{q}"] = torch.ones(W, dtype=torch.bfloat16, device=device)
            t[f"{p}canon{q}"] = rnd(W, taps, scale=0.1)
            t[f"{p}hc{q}.in"] = torch.full((S,), 1.0 / S, dtype=torch.bfloat16, device=device)
            t[f"{p}hc{q}.out"] = torch.full((S,), 0.5, dtype=torch.bfloat16, device=device)
            t[f"{p}hc{q}.mix"] = torch.eye(S, dtype=torch.bfloat16, device=device)
        if lay["type"] == "mamba2":
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            t[p + "mix.in"] = rnd(2 * inner + 2 * gn + m["heads"], W, scale=W ** -0.5)
            t[p + "mix.o"] = rnd(W, inner, scale=inner ** -0.5)
            t[p + "mix.conv"] = rnd(inner + 2 * gn, m["conv"], scale=0.3)
            t[p + "mix.conv.b"] = rnd(inner + 2 * gn, scale=0.1)
            t[p + "mix.dt_bias"] = rnd(m["heads"], scale=0.5)
            t[p + "mix.A_log"] = rnd(m["heads"], scale=0.5)
            t[p + "mix.D"] = rnd(m["heads"])
            t[p + "mix.norm"] = torch.ones(inner, dtype=torch.bfloat16, device=device)
        else:
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = rnd(H * D, W, scale=W ** -0.5), rnd(G * D, W, scale=W ** -0.5), rnd(G * V, W, scale=W ** -0.5)
            t[p + "mix.g"], t[p + "mix.o"] = rnd(H, W, scale=W ** -0.5), rnd(W, H * V, scale=(H * V) ** -0.5)
        if lay["mlp"]:
            ff = lay["mlp"]["ff"]
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = rnd(ff, W, scale=W ** -0.5), rnd(ff, W, scale=W ** -0.5), rnd(W, ff, scale=ff ** -0.5)
    return t.__getitem__


def _events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def _linear_weights(model: LayeredModel) -> int:
    """weights of the linear layers a token goes through (of a mixture of experts: the router, the chosen experts, the shared one)"""
    n = sum(L[k].numel() for L in model.layers for k in ("w_in", "w_o", "w_gu", "w_down", "w_router", "w_sup", "w_sdown", "rg1", "rg2", "w_uq", "w_ukT", "w_uv", "w_up", "w_ro", "w_gates") if k in L)
    for L in model.layers:
        if "w_eup" in L:
            n += L["spec"].ff.top * (L["w_eup"][0].numel() + L["w_edown"][0].numel())
    return n


# ---- cost model: algorithmic bytes and FLOPs of one operator call, from the shapes the timeline recorded ---------------------------
def _cost(name: str, shapes, scal, scen: dict, kw: dict = None):
    kw = kw or {}
    sh = [s for s in shapes if s is not None]
    by = lambda s: int(np.prod(s[0])) * s[1]
    if name == "depth_norm":      # x_cur, out1, w1 positional; the branches, the earlier results and the outputs by keyword
        rows = kw["rows"][0][0] if isinstance(kw.get("rows"), tuple) else sh[0][0][0]
        W = sh[0][0][1]
        reads = 1 + sum(1 for n in ("y1", "y2") if isinstance(kw.get(n), tuple)) + (kw.get("n_prev", 0) if isinstance(kw.get("dwa"), tuple) else 0)
        writes = sum(1 for n in ("hist_out", "x_out") if isinstance(kw.get(n), tuple)) if isinstance(kw.get("y1"), tuple) else 0
        outs = sum(s[1] for s in (shapes[1], kw.get("out2")) if isinstance(s, tuple))
        return rows * W * (4 * (reads + writes) + outs), 0.0, "hbm"
    if name in ("attn_prep", "attn_prep_ex"):     # the projection row in, q back, k and v rows to the pool (the pools are not streamed)
        d = scen.get("attn_desc")
        T, ld = sh[0][0]
        if name == "attn_prep_ex" and d is not None:
            return T * (ld + d.H * d.D + d.G * (d.D + d.V)) * 4, 0.0, "hbm"
        return T * ld * 4 * 2, 0.0, "hbm"
    if name in ("linear", "linear_gated", "linear_act"):
        (xs, xe), (ws, _), (ys, ye) = sh[0], sh[1], sh[2]
        M, K, N = xs[0], xs[1], ws[0]
        return M * K * xe + N * K * 2 + int(np.prod(ys)) * ye, 2.0 * M * N * K, "tensor"
    if name == "moe_linear":      # x, w [E, N, K], ids, (order, offs), out; scal: x_div, pairs, act
        (xs, xe), (ws, _) = sh[0], sh[1]
        pairs = scal[1]
        E, N, K = ws
        (os_, oe) = sh[-1]
        rows_in = pairs if scal[0] == 0 else xs[0]
        w_read = min(E, pairs) * N * K * 2           # every expert that has a pair streams its weight once
        return rows_in * K * xe + w_read + pairs * N * oe, 2.0 * pairs * N * K, "tensor"
    if name == "retention":       # the projection row in, the gated result out, the state of every entry read and written; recurrence + chunk products
        d = scen["ret_desc"]
        T, ld = sh[0][0]
        B = scen["entries"]
        flops = 2.0 * T * d.H * (3 * d.D * d.V if scen["prefill"] else 2 * d.D * d.V)      # state update, output (chunked: + the local state), without the chunk's own scores
        if scen["prefill"]:
            flops += 2.0 * T * d.H * 32 * (d.D + d.V)                                       # on average 32 of the chunk's 64 keys are at or before a token
        return T * (ld * 4 + d.H * d.V * sh[2][1]) + 2 * B * d.H * d.D * d.V * 4, flops, "f32" if scen["prefill"] else "hbm"
    if name == "latent_gather":   # pool rows in, latents out in the activation type
        (rows, R), es = sh[-1][0], sh[-1][1]
        return rows * R * (4 + es), 0.0, "hbm"
    if name == "head_linear":     # x, w [H, N, K], out
        (xs, xe), (ws, _), (os_, oe) = sh[0], sh[1], sh[2]
        H, N, K = ws
        return xs[0] * H * K * xe + H * N * K * 2 + xs[0] * H * N * oe, 2.0 * xs[0] * H * N * K, "tensor"
    if name == "latent_prep":     # projection row and query row in, pool row, rotated query parts and unrotated parts out
        (T, ldp), (_, ldq) = sh[0][0], sh[1][0]
        return T * (ldp + 2 * ldq) * 4, 0.0, "hbm"
    if name == "post_norm":       # x (+ result + gate logits) in, x and the activation rows out
        rows = kw["rows"][0][0] if isinstance(kw.get("rows"), tuple) else sh[0][0][0]
        W = sh[0][0][1]
        reads = 1 + sum(1 for n in ("y", "zg") if isinstance(kw.get(n), tuple))
        outs = sum(kw[n][1] for n in ("x_out", "a_out", "a_shift_out") if isinstance(kw.get(n), tuple))
        return rows * W * (4 * reads + outs), 0.0, "hbm"
    if name == "token_shift":
        (T, W), outs = sh[0][0], sum(s[1] for s in sh[3:])
        return T * W * (4 + outs), 0.0, "hbm"
    if name == "moe_table_route":
        T, top = scal[0], scal[2]
        return T * 4 + T * top * 12, 0.0, "hbm"
    if name in ("attn", "attn_ex"):
        if name == "attn_ex":
            d = scen["attn_desc"]
            T, H, G, D, V = sh[0][0][0], d.H, d.G, d.D, d.V
        else:
            T, H, G, D, V = sh[0][0][0], scal[0], scal[1], scal[2], scal[3]
        keys = scen["visible_keys"]                              # sum over the step's tokens of the keys each one sees
        kv_once = scen["kv_rows_touched"] * G * (D if getattr(d, "latent_v", 0) else D + V) * 4 if name == "attn_ex" else scen["kv_rows_touched"] * G * (D + V) * 4   # every visible K / V row once
        return kv_once + T * H * (D + V) * 4, 2.0 * keys * H * (D + V), "f32" if scen["prefill"] else "hbm"
    if name == "min_gru":         # three f32 columns of the projection row per channel in, the gated state out; the entries' states read and written
        T, C, oe = sh[0][0][0], scal[3], sh[-1][1]
        return T * C * (12 + oe) + 2 * scen["entries"] * C * 4, 12.0 * T * C, "hbm"
    if name == "rg_lru":          # u, two gate columns and the y column in, the gated state out
        (T, C), oe = sh[0][0], sh[-1][1]
        return T * C * (16 + oe) + 2 * scen["entries"] * C * 4, 16.0 * T * C, "hbm"
    if name == "causal_conv_ex":  # the input column in, the result out in f32 and in the activation type
        (T, C) = sh[0][0]
        return T * C * sum(s[1] for s in sh if s[0] == (T, C)), 0.0, "hbm"
    if name == "branch_norm":     # x and the branches in; x and / or the activation rows out
        rows = kw["rows"][0][0] if isinstance(kw.get("rows"), tuple) else sh[0][0][0]
        W = sh[0][0][1]
        reads = 2 + (1 if isinstance(kw.get("y2"), tuple) else 0)
        outs = sum(kw[n][1] for n in ("x_out", "a_out") if isinstance(kw.get(n), tuple))
        return rows * W * (4 * reads + outs), 0.0, "hbm"
    if name == "embed_bigram":    # two bf16 table rows in, the residual and the activation rows out
        (T, W) = sh[-2][0] if len(sh) >= 2 else sh[-1][0]
        return T * W * (4 + 4 + sh[-1][1]), 0.0, "hbm"
    if name == "ssm_scan":
        T, (H, V, N, G) = sh[0][0][0], scal[2:6]
        B = scen["entries"]
        return T * (2 * H * V + 2 * G * N + H) * 4 + T * H * V * 4 + 2 * B * H * N * V * 4, 4.0 * T * H * V * N, "f32" if scen["prefill"] else "hbm"
    # elementwise / normalising operators: every tensor argument once (in-place stream update: read + write)
    total = sum(by(s) for s in sh)
    if name == "hc_norm" and len(sh) >= 2 and shapes[1] is not None:
        total += by(sh[0])
    return total, 0.0, "hbm"


def _roof_us(bytes_, flops, kind, pk) -> float:
    t_mem = bytes_ / (pk["hbm_gbs"] * 1e9)
    t_fl = flops / ((pk["bf16_tflops"] if kind == "tensor" else F32_FMA_TFLOPS_NOMINAL) * 1e12) if kind in ("tensor", "f32") else 0.0
    return max(t_mem, t_fl) * 1e6


def kernel_table(model: LayeredModel, eng: Engine, run, scen: dict, pk) -> List[dict]:
    """runs `run()` (one engine step) with the operator timeline on and sums time and cost per operator (linear layers per shape)"""
    graphs = model.use_graphs
    model.use_graphs = False
    try:
        seqops.timeline = []
        run()
        torch.cuda.synchronize()
        tl, seqops.timeline = seqops.timeline, None
    finally:
        seqops.timeline = None
        model.use_graphs = graphs
    agg: Dict[str, dict] = {}
    for name, shapes, scal, e0, e1, kw in tl:
        key = name
        if name in ("linear", "linear_gated", "linear_act"):
            sh = [s for s in shapes if s is not None]
            key = f"{name} M={sh[0][0][0]} N={sh[1][0][0]} K={sh[0][0][1]}"
        elif name == "moe_linear":
            sh = [s for s in shapes if s is not None]
            key = f"moe_linear pairs={scal[1]} E={sh[1][0][0]} N={sh[1][0][1]} K={sh[1][0][2]}"
        b, f, kind = _cost(name, shapes, scal, scen, kw)
        a = agg.setdefault(key, dict(op=key, calls=0, us=0.0, bytes=0, flops=0.0, roof_us=0.0, bound=kind))
        a["calls"] += 1
        a["us"] += e0.elapsed_time(e1) * 1e3
        a["bytes"] += b
        a["flops"] += f
        a["roof_us"] += _roof_us(b, f, kind, pk)
    rows = []
    for a in agg.values():
        a["frac_of_roofline"] = round(a["roof_us"] / a["us"], 4) if a["us"] > 0 else None
        a["us"], a["roof_us"] = round(a["us"], 1), round(a["roof_us"], 1)
        rows.append(a)
    rows.sort(key=lambda r: -r["us"])
    return rows


# ---- the design's arm ----------------------------------------------------------------------------------------------------------------
def bench_layered(design: str, size: str, pk, S: int = 4096, ctx: int = 1024, batches=(1, 4), steps: int = 32, dtype: str = "bfloat16") -> dict:
    from . import registry
    sz = SIZES[size]
    dev = torch.device("cuda", torch.cuda.current_device())
    if design.lower() == "fenorax":
        cfg = fenorax_config(sz)
        model = LayeredModel(registry.LAYERED["Fenorax"](cfg), random_tensors(cfg, dev), dev, dtype)
    elif design.lower() == "gemosun":
        cfg = gemosun_config(sz)
        model = LayeredModel(registry.LAYERED["Gemosun"](cfg), random_tensors_gemosun(cfg, dev), dev, dtype)
    elif design.lower() == "teselix":
        cfg = teselix_config(sz)
        model = LayeredModel(registry.LAYERED["Teselix"](cfg), random_tensors_teselix(cfg, dev), dev, dtype)
    elif design.lower() == "pafelorn":
        cfg = pafelorn_config(sz)
        model = LayeredModel(registry.LAYERED["Pafelorn"](cfg), random_tensors_pafelorn(cfg, dev), dev, dtype)
    else:
        raise ValueError(f"no synthetic workload for design '{design}'")
    gem, tes, paf = design.lower() == "gemosun", design.lower() == "teselix", design.lower() == "pafelorn"
    pool = 16 if gem else 0
    desc0 = next((L["desc"] for L in model.layers if isinstance(L.get("desc"), seqops.AttnDesc)), None)
    rdesc0 = next((L["desc"] for L in model.layers if isinstance(L.get("desc"), seqops.RetentionDesc)), None)
    Bmax = max(batches)
    eng = Engine(model, max_tokens=max(S, Bmax * (ctx + steps + 64)) + 64, max_seqs=Bmax, max_step_tokens=max(S, 2048), prefill_chunk=S)
    rng = np.random.default_rng(3)
    prompt = rng.integers(0, sz["vocab"], S).tolist()
    out = {"size": size, "config": {k: sz[k] for k in sz}, "layers": [l["type"] + ("+" + l["mlp"].get("kind", "ff") if l["mlp"] else "") for l in cfg["layers"]],
           "streams": cfg.get("streams", 1), "linear_weights": _linear_weights(model), "weight_bytes": model.weight_bytes}
    if gem or tes or paf:
        r = cfg["layers"][1]["mlp"]
        out["experts"] = {"experts": r["router"]["experts"], "top": r["router"]["top"], "ff": r["expert"]["ff"], "shared_ff": r["shared"]["ff"], "groups": r["router"].get("groups")}
    lin_flops_tok = 2.0 * (_linear_weights(model) + 0)

    # prefill: whole prompt in one step, logits of the last token, device timed; then through run_entries (host arrays in, logits out)
    def prefill_once():
        eng._forward([("p", prompt, [S - 1])])
        eng.release("p")

    for _ in range(3):
        prefill_once()
    torch.cuda.synchronize()
    e0, e1 = _events()
    reps = 5
    e0.record()
    for _ in range(reps):
        prefill_once()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    e0, e1 = _events()
    e0.record()
    for _ in range(reps):
        eng.run_entries([{"id": "p", "tokens": prompt, "want": [S - 1]}], end=["p"])
    e1.record()
    torch.cuda.synchronize()
    ms_e2e = e0.elapsed_time(e1) / reps
    out["prefill"] = {"prompt_tokens": S, "ms": round(ms, 3), "tokens_per_s": round(S / ms * 1e3, 1), "e2e_tokens_per_s": round(S / ms_e2e * 1e3, 1),
                      "linear_TFLOPs": round(lin_flops_tok * S / (ms * 1e-3) / 1e12, 1)}
    chunk = sz["chunk"]
    pos = np.arange(S)
    if gem:     # window of `chunk` positions plus one pooled entry per block of 16 wholly before it
        vis = np.minimum(pos + 1, chunk) + np.maximum(0, (pos - chunk + 1) // pool)
        scen = dict(prefill=True, entries=1, visible_keys=int(vis.sum()), kv_rows_touched=S + S // pool, attn_desc=desc0)
    elif paf:   # a sliding window of `chunk` positions (the few kept first positions of one layer are not counted)
        scen = dict(prefill=True, entries=1, visible_keys=int(np.minimum(pos + 1, chunk).sum()), kv_rows_touched=S, attn_desc=desc0)
    elif tes:   # every earlier position; a step of portions attends over per-head keys projected from the gathered latents
        descx = next((L["desc_x"] for L in model.layers if "desc_x" in L), desc0)
        scen = dict(prefill=True, entries=1, visible_keys=int((pos + 1).sum()), kv_rows_touched=S, attn_desc=descx, ret_desc=rdesc0)
    else:
        scen = dict(prefill=True, entries=1, visible_keys=int((pos - (pos // chunk) * chunk + 1).sum()), kv_rows_touched=S, attn_desc=desc0)
    out["prefill"]["kernels"] = kernel_table(model, eng, prefill_once, scen, pk)

    # decode: B requests of ctx tokens, then one token each per step
    out["decode"] = []
    for B in batches:
        ids = [f"d{b}" for b in range(B)]
        for r in ids:
            eng._forward([(r, rng.integers(0, sz["vocab"], ctx).tolist(), [])])
        nxt = [[1]] * B

        def dec_step():
            eng._forward([(r, t, [0]) for r, t in zip(ids, nxt)], sample=True)

        for _ in range(4):
            dec_step()
        torch.cuda.synchronize()
        e0, e1 = _events()
        e0.record()
        for _ in range(steps):
            dec_step()
        e1.record()
        torch.cuda.synchronize()
        msd = e0.elapsed_time(e1) / steps
        # end to end: token ids come back to the host every step and go in again (pinned upload inside the step)
        e0, e1 = _events()
        e0.record()
        for _ in range(steps):
            dec_step()
            nxt = [[int(t)] for t in model.last_ids.cpu().tolist()]
        e1.record()
        torch.cuda.synchronize()
        msd_e2e = e0.elapsed_time(e1) / steps
        # weights a step streams: all of them but the experts no token of the step chose (at most B * top of a layer's experts are touched)
        touched = model.weight_bytes
        for L in model.layers:
            if "w_eup" in L:
                E_, per = L["w_eup"].shape[0], (L["w_eup"][0].numel() + L["w_edown"][0].numel()) * 2
                touched -= (E_ - min(E_, B * L["spec"].ff.top)) * per
        row = {"batch": B, "context": ctx, "ms_per_step": round(msd, 4), "tokens_per_s": round(B / msd * 1e3, 1), "e2e_tokens_per_s": round(B / msd_e2e * 1e3, 1),
               "weight_bytes_touched": touched, "weight_GBs": round(touched / (msd * 1e-3) / 1e9, 1),
               "frac_hbm_weights_only": round(touched / (msd * 1e-3) / 1e9 / pk["hbm_gbs"], 3)}
        held = eng.cache.live[ids[0]].n_tokens
        lo = (held // chunk) * chunk
        seen = (min(held + 1, chunk) + max(0, (held - chunk + 1) // pool)) if gem else (held + 1 if tes else (min(held + 1, chunk) if paf else held - lo + 1))
        scen = dict(prefill=False, entries=B, visible_keys=B * seen, kv_rows_touched=B * seen, attn_desc=desc0, ret_desc=rdesc0)
        row["kernels"] = kernel_table(model, eng, dec_step, scen, pk)
        out["decode"].append(row)
        for r in ids:
            eng.release(r)
    flags = seqops.error_flags()
    if flags:
        raise RuntimeError(f"device error flags {flags:#x}")
    out["launches"] = seqops.launch_count()
    del eng, model
    torch.cuda.empty_cache()
    return out


# ---- the dense-attention decoder of equal size ---------------------------------------------------------------------------------------
def bench_decoder(size: str, pk, S: int = 4096, ctx: int = 1024, batches=(1, 4), steps: int = 32, scheme: str = "Q8_0") -> dict:
    """Same width, heads, feed-forward size, vocabulary and layer count; every layer is attention + feed-forward; weights Q8_0."""
    import ctypes as C

    from . import decode, ops
    sz = SIZES[size]
    cfg = decode.ModelConfig(f"dense-{size}", sz["width"], 4, sz["heads"], sz["kv_heads"], sz["dim"], sz["ff"], sz["vocab"], 10000.0)
    client = ops.B200Client(torch.cuda.current_device())
    rng = np.random.default_rng(3)
    out = {"size": size, "scheme": scheme, "layers": 4}
    d = decode.Decoder(client, cfg, scheme, batch=1, max_ctx=S + 16)
    lin_w = sum(ln.w.N * ln.w.K for lay in d.layers for key in ("qkv", "o", "gu", "down") for ln in lay[key])
    out["linear_weights"], out["weight_bytes"] = lin_w, d.weight_bytes
    prompt = rng.integers(0, cfg.vocab, S)
    for _ in range(2):
        d.prefill(prompt)
    torch.cuda.synchronize()
    e0, e1 = _events()
    reps = 3
    e0.record()
    for _ in range(reps):
        d.prefill(prompt)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    out["prefill"] = {"prompt_tokens": S, "ms": round(ms, 3), "tokens_per_s": round(S / ms * 1e3, 1), "linear_TFLOPs": round(2.0 * lin_w * S / (ms * 1e-3) / 1e12, 1),
                      "note": "projections on the tcgen05 dequant-GEMM, attention of the prompt in torch SDPA (f16)"}
    # like kernels, timed alone: the gate|up GEMM at M = S, the gate|up matvec at M = 1, the norm at M = S
    kern = []
    lay = d.layers[0]
    gu = lay["gu"][0]
    x = torch.randn((S, cfg.hidden), device=client.device)
    y = torch.empty((S, gu.w.N), device=client.device)
    ws = gu.w.workspace(S)
    for _ in range(2):
        client.quant_matmul(x, gu.w, out=y, workspace=ws)
    e0, e1 = _events()
    e0.record()
    for _ in range(5):
        client.quant_matmul(x, gu.w, out=y, workspace=ws)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / 5
    fl = 2.0 * S * gu.w.N * gu.w.K
    roof = max(fl / (pk["bf16_tflops"] * 1e12), (gu.w.canonical_bytes + S * gu.w.K * 4 + S * gu.w.N * 4) / (pk["hbm_gbs"] * 1e9)) * 1e6
    kern.append({"op": f"dequant GEMM gate|up M={S} N={gu.w.N} K={gu.w.K} (staging + tcgen05)", "us": round(us, 1), "roof_us": round(roof, 1), "frac_of_roofline": round(roof / us, 4),
                 "bound": "tensor"})
    # residual add + RMS norm at M = S (the like kernel of the stream update + grouped norm): reads h, delta, writes h', normed
    Hd = cfg.hidden
    hin, dl, hout, xn = (torch.randn((S, Hd), device=client.device) for _ in range(4))
    L_, P_ = ops.lib(), (lambda t_: C.c_void_p(t_.data_ptr()))
    st_ = ops._stream_ptr(client.device)

    def norm_once():
        ops._check(L_.b200q_add_rmsnorm_quant(P_(hin), P_(dl), P_(hout), P_(lay["attn_norm"]), C.c_float(cfg.eps), C.c_int64(Hd), C.c_int64(S), None, P_(xn), st_))

    for _ in range(3):
        norm_once()
    e0, e1 = _events()
    e0.record()
    for _ in range(10):
        norm_once()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / 10
    by = 4 * S * Hd * 4
    kern.append({"op": f"residual add + RMS norm M={S} W={Hd}", "us": round(us, 1), "roof_us": round(by / (pk['hbm_gbs'] * 1e9) * 1e6, 1),
                 "frac_of_roofline": round(by / (pk["hbm_gbs"] * 1e9) * 1e6 / us, 4), "bound": "hbm"})
    del d, x, y, ws, hin, dl, hout, xn
    torch.cuda.empty_cache()
    out["decode"] = []
    for B in batches:
        d = decode.Decoder(client, cfg, scheme, batch=B, max_ctx=ctx + 3 * steps + 64)
        d.capture()
        d.reset([1] * B)
        for b in range(B):
            d.prefill(rng.integers(0, cfg.vocab, ctx), seq=b)
        for _ in range(4):
            d.replay()
        torch.cuda.synchronize()
        e0, e1 = _events()
        e0.record()
        for _ in range(steps):
            d.replay()
        e1.record()
        torch.cuda.synchronize()
        msd = e0.elapsed_time(e1) / steps
        row = {"batch": B, "context": ctx, "ms_per_step": round(msd, 4), "tokens_per_s": round(B / msd * 1e3, 1), "weight_GBs": round(d.weight_bytes / (msd * 1e-3) / 1e9, 1),
               "frac_hbm_weights_only": round(d.weight_bytes / (msd * 1e-3) / 1e9 / pk["hbm_gbs"], 3), "launches_per_step": d.launches_per_step()}
        if B == 1:
            # attention of one decoded token over the context, every layer, timed alone (K / V rows of the context once per kv head)
            st = ops._stream_ptr(client.device)
            for lay in d.layers:
                d._attention(lay, st)
            torch.cuda.synchronize()
            e0, e1 = _events()
            e0.record()
            for _ in range(5):
                for lay in d.layers:
                    d._attention(lay, st)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (5 * len(d.layers))
            held = int(d._host_pos)
            by = held * cfg.n_kv_heads * cfg.head_dim * 2 * 4
            kern.append({"op": f"attention decode, {held} keys, H={cfg.n_heads} G={cfg.n_kv_heads} D={cfg.head_dim}", "us": round(us, 2), "roof_us": round(by / (pk['hbm_gbs'] * 1e9) * 1e6, 2),
                         "frac_of_roofline": round(by / (pk["hbm_gbs"] * 1e9) * 1e6 / us, 4), "bound": "hbm"})
            gu = d.layers[0]["gu"][0]
            xq = client.quantize_act(torch.randn((1, gu.w.K), device=client.device))
            yv = torch.empty((1, gu.w.N), device=client.device)
            wsv = gu.w.workspace(1)
            gus = [lay["gu"][0] for lay in d.layers]
            for g_ in gus:
                client.matmul_q8(xq, 1, g_.w, out=yv, workspace=wsv)
            e0, e1 = _events()
            e0.record()
            for _ in range(5):
                for g_ in gus:
                    client.matmul_q8(xq, 1, g_.w, out=yv, workspace=wsv)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (5 * len(gus))
            by = gu.w.canonical_bytes
            kern.append({"op": f"matvec gate|up M=1 N={gu.w.N} K={gu.w.K} ({scheme})", "us": round(us, 2), "roof_us": round(by / (pk['hbm_gbs'] * 1e9) * 1e6, 2),
                         "frac_of_roofline": round(by / (pk["hbm_gbs"] * 1e9) * 1e6 / us, 4), "bound": "hbm"})
        out["decode"].append(row)
        d.graph = None
        del d
        torch.cuda.empty_cache()
    out["kernels"] = kern
    return out


def run(design: str, sizes: List[str], pk, pk_kind: str, S: int = 4096, ctx: int = 1024, steps: int = 32, clocks=None) -> dict:
    res = {"metric": "layered_prefill_decode_tokens_per_s", "design": design, "dtype": "bf16 activations x bf16 weights, f32 accumulate; residual, norms, scores, state f32",
           "data": "synthetic (random weights)", "peaks": {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "kind": pk_kind, "f32_fma_tflops_nominal": round(F32_FMA_TFLOPS_NOMINAL, 1)},
           "timing": "CUDA events, >= 3 warm-up runs; every prefill step streams activations larger than L2, decode weights are re-read from L2 / HBM as in serving",
           "sizes": []}
    for size in sizes:
        row = {"size": size}
        row[design.lower()] = bench_layered(design, size, pk, S=S, ctx=ctx, steps=steps)
        others = {"fenorax": [], "gemosun": ["fenorax"], "teselix": ["gemosun", "fenorax"], "pafelorn": ["gemosun", "fenorax"]}.get(design.lower(), ["fenorax"])
        for other in others:                # the closest existing layer-list models at the same sizes
            try:
                row[other] = bench_layered(other, size, pk, S=S, ctx=ctx, steps=steps)
            except Exception as ex:
                row[other] = {"error": repr(ex)[:300]}
        try:
            row["dense_decoder"] = bench_decoder(size, pk, S=S, ctx=ctx, steps=steps)
        except Exception as ex:    # the comparison arm must not take the design's numbers down
            row["dense_decoder"] = {"error": repr(ex)[:300]}
        res["sizes"].append(row)
    return res
