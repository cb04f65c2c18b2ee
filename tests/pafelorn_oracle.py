"""Plain, slow restatement of the Pafelorn layer types in torch (CPU, float64): one function per mechanism, position by position where
the mechanism is a mask or a recurrence.  Test infrastructure only: nothing here is imported by the package, and nothing of the package
is imported here.

Notation: T tokens of ONE sequence, W model width, weights as a dict name -> tensor with the checkpoint's names.

The design in short.  Sublayers come in sequence and read the residual x itself; the RMS norm sits on what a sublayer returns:
x <- x + rms(sublayer(x)) * w.  Mixers: differential attention (two soft-max maps per head over the same values, combined as
a1 - lambda a2, optionally over an earlier layer's keys and values), or two branches side by side - a windowed attention beside an
element-wise gated recurrence.  Feed-forward: dense with a polynomial-of-norms activation, or experts chosen by a soft-max router
with a correction on the choice, identity experts and a gated shared expert.  The embedding adds a row of a hashed bigram table.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ---- norms and activations ---------------------------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, eps: float, w: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension, times w when given"""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    """c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3, powers element by element, N = rms_norm without weight over the row"""
    return coef[0] * rms_norm(z, eps) + coef[1] * rms_norm(z * z, eps) + coef[2] * rms_norm(z * z * z, eps) + coef[3]


# ---- embedding ---------------------------------------------------------------------------------------------------------------------
def embed(tokens: List[int], w: Dict[str, torch.Tensor], emb: dict) -> torch.Tensor:
    rows = []
    bg = emb.get("bigram")
    for t, tok in enumerate(tokens):
        v = w["embed"][tok] * emb["scale"]
        if bg:
            r = bg["buckets"] if t == 0 else (tokens[t - 1] * bg["mul_prev"] + tok * bg["mul_cur"]) % bg["buckets"]
            v = v + w["bigram"][r]
        rows.append(v)
    return torch.stack(rows)


# ---- rotary positions --------------------------------------------------------------------------------------------------------------
def rotary_frequencies(rot: dict) -> List[float]:
    dims, base = rot["dims"], rot["base"]
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if sc and "original" in sc:      # three bands by wavelength
            wl = 2.0 * math.pi / f
            if wl > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif wl >= sc["original"] / sc["high"]:
                s = (sc["original"] / wl - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        elif sc:
            f = f / sc["factor"]
        out.append(f)
    return out


def rotate(x: torch.Tensor, rot: Optional[dict], layout: str) -> torch.Tensor:
    """x [T, heads, D]: the first rot.dims dimensions of every head turn with the position; partner of dimension 2i is 2i + 1 ("interleaved")
    or partner of i is i + dims / 2 ("half")"""
    if not rot:
        return x
    out = x.clone()
    freq = rotary_frequencies(rot)
    half = rot["dims"] // 2
    for t in range(x.shape[0]):
        for i, f in enumerate(freq):
            a, b = (2 * i, 2 * i + 1) if layout == "interleaved" else (i, i + half)
            c, s = math.cos(t * f), math.sin(t * f)
            u, v = x[t, :, a], x[t, :, b]
            out[t, :, a] = u * c - v * s
            out[t, :, b] = v * c + u * s
    return out


# ---- attention ---------------------------------------------------------------------------------------------------------------------
def visible(i: int, j: int, window: int, keep_first: int) -> bool:
    return j <= i and (window <= 0 or i - j < window or j < keep_first)


def masked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int, keep_first: int = 0, softcap: float = 0.0,
                     temp: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, Gv, V] (query head h reads key head h / (H / G), key head g reads value head g / (G / Gv)) -> [T, H, V];
    row by row: scores of the visible keys, optional soft cap, soft-max whose denominator may hold one more term exp(sink_h)"""
    T, H, _ = q.shape
    G, Gv = k.shape[1], v.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for i in range(T):
        js = [j for j in range(T) if visible(i, j, window, keep_first)]
        for h in range(H):
            g = h // (H // G)
            s = (k[js, g] @ q[i, h]) * scale
            if temp is not None:
                s = s * temp[h]
            if softcap > 0:
                s = softcap * torch.tanh(s / softcap)
            mx = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - mx)
            den = e.sum() + (torch.exp(sink[h] - mx) if sink is not None else 0.0)
            out[i, h] = (e / den) @ v[js, g // (G // Gv)]
    return out


def project(h: torch.Tensor, w: Dict[str, torch.Tensor], name: str, bias: bool = False) -> torch.Tensor:
    y = h @ w[name].T
    return y + w[name + ".b"] if bias else y


def differential_attention(h, w, p, m, eps, kv_store, layer):
    """two maps per head, rows of q / k laid out head by head as [map 1 | map 2]; the maps share the head's values"""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rotate(rms_norm(project(h, w, p + "q", True).view(T, 2 * H, D), eps, w[p + "q.norm"]), m.get("rot"), "half")
    if m.get("kv_from") is not None:
        k, v = kv_store[m["kv_from"]]
    else:
        k = rotate(rms_norm(project(h, w, p + "k", True).view(T, 2 * G, D), eps, w[p + "k.norm"]), m.get("rot"), "half")
        v = project(h, w, p + "v", True).view(T, G, V)
        kv_store[layer] = (k, v)
    lam = torch.exp((w[p + "lq1"] * w[p + "lk1"]).sum()) - torch.exp((w[p + "lq2"] * w[p + "lk2"]).sum()) + m["diff"]
    window = (m.get("mask") or {}).get("size", 0)
    maps = []
    for mp in (0, 1):      # map mp of head h is row 2 h + mp of q and row 2 g + mp of k
        maps.append(masked_attention(q[:, mp::2], k[:, mp::2], v, m["scale"], window))
    o = rms_norm(maps[0] - lam * maps[1], eps) * (1.0 - m["diff"])
    return project(o.reshape(T, H * V), w, p + "o")


def branch_attention(h, w, p, m, eps, second: bool):
    """left branch of a two-branch mixer.  first form: biases, per-head q / k norm, sink and temperature per head.  second form: q / k norm over the
    whole projection, soft cap, kept first tokens, element-wise sigmoid gate on the heads' outputs"""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    mask = m.get("mask") or {}
    if not second:
        q = rms_norm(project(h, w, p + "q", True).view(T, H, D), eps, w[p + "q.norm"])
        k = rms_norm(project(h, w, p + "k", True).view(T, G, D), eps, w[p + "k.norm"])
        v = project(h, w, p + "v", True).view(T, G, V)
    else:
        q = rms_norm(project(h, w, p + "q"), eps, w[p + "q.norm"]).view(T, H, D)
        k = rms_norm(project(h, w, p + "k"), eps, w[p + "k.norm"]).view(T, G, D)
        v = project(h, w, p + "v").view(T, G, V)
    q, k = rotate(q, m.get("rot"), "interleaved"), rotate(k, m.get("rot"), "interleaved")
    if not second:
        o = masked_attention(q, k, v, m["scale"], mask.get("size", 0), temp=w[p + "temp"], sink=w[p + "sink"])
        return project(o.reshape(T, H * V), w, p + "o", True)
    o = masked_attention(q, k, v, m["scale"], mask.get("size", 0), keep_first=mask.get("keep_first", 0), softcap=m.get("softcap", 0.0))
    o = o.reshape(T, H * V) * torch.sigmoid(project(h, w, p + "g"))
    return project(o, w, p + "o")


# ---- recurrences -------------------------------------------------------------------------------------------------------------------
def min_gru(h, w, p):
    z = torch.sigmoid(project(h, w, p + "z", True))
    u = project(h, w, p + "x", True)
    g = project(h, w, p + "g")
    S = torch.zeros(u.shape[1], dtype=h.dtype)
    rows = []
    for t in range(h.shape[0]):
        cand = torch.where(u[t] >= 0, u[t] + 0.5, torch.sigmoid(u[t]))
        S = (1.0 - z[t]) * S + z[t] * cand
        rows.append(S * g[t] * torch.sigmoid(g[t]))
    return project(torch.stack(rows), w, p + "o")


def causal_conv(x: torch.Tensor, cw: torch.Tensor, cb: torch.Tensor) -> torch.Tensor:
    """x [T, C], cw [C, taps] whose last column meets the current token; zeros before the start"""
    T, taps = x.shape[0], cw.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        acc = cb.clone()
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                acc = acc + cw[:, j] * x[s]
        out[t] = acc
    return out


def rg_lru(h, w, p, m):
    y = gelu_tanh(project(h, w, p + "y", True))
    u = causal_conv(project(h, w, p + "x", True), w[p + "conv"], w[p + "conv.b"])
    nb = m["blocks"]
    bw = m["width"] // nb
    sp = torch.log1p(torch.exp(w[p + "lam"]))
    S = torch.zeros(m["width"], dtype=h.dtype)
    rows = []
    for t in range(h.shape[0]):
        r = torch.cat([torch.sigmoid(w[p + "ra"][b] @ u[t, b * bw:(b + 1) * bw] + w[p + "ra.b"][b]) for b in range(nb)])
        i = torch.cat([torch.sigmoid(w[p + "ri"][b] @ u[t, b * bw:(b + 1) * bw] + w[p + "ri.b"][b]) for b in range(nb)])
        a = torch.exp(-8.0 * r * sp)
        S = a * S + torch.sqrt(1.0 - a * a) * i * u[t]
        rows.append(S * y[t])
    return project(torch.stack(rows), w, p + "o")


# ---- feed-forward ------------------------------------------------------------------------------------------------------------------
def expert(h, w, p, limit):
    g = torch.clamp(project(h, w, p + "gate"), max=limit)
    u = torch.clamp(project(h, w, p + "up"), -limit, limit)
    return project(g * torch.sigmoid(1.702 * g) * (u + 1.0), w, p + "down")


def routed_experts(h, w, p, f):
    r = f["router"]
    E, top = r["experts"], r["top"]
    s = torch.softmax(project(h, w, p + "router"), -1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        choice = (s[t] + w[p + "correction"]).tolist()
        picked = sorted(range(len(choice)), key=lambda e: (-choice[e], e))[:top]
        tot = sum(s[t, e] for e in picked) + 1e-20
        for e in picked:
            out[t] += (s[t, e] / tot) * (h[t] if e >= E else expert(h[t:t + 1], w, p + f"e{e}.", f["expert"]["limit"])[0])
    if f.get("shared"):
        out = out + torch.sigmoid(project(h, w, p + "shared.sg")) * expert(h, w, p + "shared.", f["shared"]["limit"])
    return out


# ---- the model ---------------------------------------------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None, dtype=F64) -> torch.Tensor:
    """logits [T, vocab] of one sequence from position 0"""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = embed(tokens, w, cfg["embedding"])
    kv_store = {}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        if lay["type"] == "attention":
            y = differential_attention(x, w, p + "mix.", m, eps, kv_store, i)
        elif lay["type"] == "parallel":
            y = m["left_scale"] * branch_attention(x, w, p + "mix.left.", m["left"], eps, False) + m["right_scale"] * min_gru(x, w, p + "mix.right.")
        else:
            y = 0.5 * (rms_norm(branch_attention(x, w, p + "mix.left.", m["left"], eps, True), eps, w[p + "mix.left.out"])
                       + rms_norm(rg_lru(x, w, p + "mix.right.", m["right"]), eps, w[p + "mix.right.out"]))
        x = x + rms_norm(y, eps, w[p + "norm1"])
        f = lay.get("mlp")
        if f is not None:
            if f["kind"] == "dense":
                r = project(polynorm(project(x, w, p + "mlp.up"), w[p + "mlp.act"], eps), w, p + "mlp.down")
            else:
                r = routed_experts(x, w, p + "mlp.", f)
            x = x + rms_norm(r, eps, w[p + "norm2"])
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = project(rms_norm(x, eps, w["final.norm"]), w, "head")
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits


# ---- random checkpoints ------------------------------------------------------------------------------------------------------------
def random_model(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """random weights that are exact in bfloat16 (so that float32 runs of the framework see the same numbers)"""
    gen = torch.Generator().manual_seed(seed)
    W, Vc = cfg["width"], cfg["vocab"]
    P: Dict[str, torch.Tensor] = {}

    def rnd(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=gen) * std + mean).to(torch.bfloat16).to(torch.float32)

    def lin(name, o, i, bias=False, gain=1.0):
        P[name] = rnd(o, i, std=gain / math.sqrt(i))
        if bias:
            P[name + ".b"] = rnd(o, std=0.3)

    P["embed"] = rnd(Vc, W)
    bg = cfg["embedding"].get("bigram")
    if bg:
        P["bigram"] = rnd(bg["buckets"] + 1, W, std=0.7)
    P["head"] = rnd(Vc, W, std=1.0 / math.sqrt(W))
    P["final.norm"] = rnd(W, std=0.2, mean=1.0)

    def attention(p, m, kind):
        H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        maps = 2 if kind == "attention" else 1
        b = kind != "parallel_2"
        own_kv = m.get("kv_from") is None
        lin(p + "q", H * maps * D, W, b, 2.0)
        if own_kv:
            lin(p + "k", G * maps * D, W, b, 2.0)
            lin(p + "v", G * V, W, b)
        if kind == "parallel_2":
            P[p + "q.norm"], P[p + "k.norm"] = rnd(H * D, std=0.3, mean=1.0), rnd(G * D, std=0.3, mean=1.0)
            lin(p + "g", H * V, W)
        else:
            P[p + "q.norm"] = rnd(D, std=0.3, mean=1.0)
            if own_kv:
                P[p + "k.norm"] = rnd(D, std=0.3, mean=1.0)
        if kind == "attention":
            for nm in ("lq1", "lk1", "lq2", "lk2"):
                P[p + nm] = rnd(D, std=0.4 / math.sqrt(D) ** 0.5)
        if kind == "parallel":
            P[p + "temp"], P[p + "sink"] = rnd(H, std=0.3, mean=1.0), rnd(H, std=1.5)
        lin(p + "o", W, H * V, kind == "parallel")

    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        P[p + "norm1"] = rnd(W, std=0.2, mean=0.7)
        if lay["type"] == "attention":
            attention(p + "mix.", m, "attention")
        else:
            attention(p + "mix.left.", m["left"], lay["type"])
            C = m["right"]["width"]
            r = p + "mix.right."
            if lay["type"] == "parallel":
                lin(r + "z", C, W, True)
                lin(r + "x", C, W, True)
                lin(r + "g", C, W)
            else:
                nb, taps = m["right"]["blocks"], m["right"]["conv"]
                bw = C // nb
                lin(r + "y", C, W, True)
                lin(r + "x", C, W, True)
                P[r + "conv"], P[r + "conv.b"] = rnd(C, taps, std=0.5), rnd(C, std=0.2)
                for nm in ("ra", "ri"):
                    P[r + nm], P[r + nm + ".b"] = rnd(nb, bw, bw, std=1.0 / math.sqrt(bw)), rnd(nb, bw, std=0.5)
                P[r + "lam"] = rnd(C, std=1.0, mean=-2.0)
                P[p + "mix.left.out"], P[p + "mix.right.out"] = rnd(W, std=0.2, mean=1.0), rnd(W, std=0.2, mean=1.0)
            lin(r + "o", W, C)
        f = lay.get("mlp")
        if f is None:
            continue
        P[p + "norm2"] = rnd(W, std=0.2, mean=0.7)
        if f["kind"] == "dense":
            lin(p + "mlp.up", f["ff"], W)
            lin(p + "mlp.down", W, f["ff"])
            P[p + "mlp.act"] = rnd(4, std=0.5, mean=0.3)
        else:
            rt = f["router"]
            n_out = rt["experts"] + rt.get("identity", 0)
            lin(p + "mlp.router", n_out, W, gain=2.0)
            P[p + "mlp.correction"] = rnd(n_out, std=0.1)
            for e in range(rt["experts"]):
                lin(p + f"mlp.e{e}.gate", f["expert"]["ff"], W, gain=2.0)
                lin(p + f"mlp.e{e}.up", f["expert"]["ff"], W, gain=2.0)
                lin(p + f"mlp.e{e}.down", W, f["expert"]["ff"])
            if f.get("shared"):
                lin(p + "mlp.shared.gate", f["shared"]["ff"], W, gain=2.0)
                lin(p + "mlp.shared.up", f["shared"]["ff"], W, gain=2.0)
                lin(p + "mlp.shared.down", W, f["shared"]["ff"])
                lin(p + "mlp.shared.sg", 1, W)
    return P


def write_checkpoint(folder: str, cfg: dict, P: Dict[str, torch.Tensor]) -> None:
    """config.json + model.safetensors (bfloat16 tensors; header = 8-byte length + JSON, then the data)"""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    head, blobs, off = {}, [], 0
    for name, t in P.items():
        raw = t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        head[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(head).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
