"""Plain, slow restatement of the Teselix layer types in torch (CPU, float64): one function per mechanism, position by position
where the mechanism is a mask or a recurrence.  Test infrastructure only: nothing here is imported by the package, and nothing of
the package is imported here.

Notation: T tokens of ONE sequence, W model width, weights as a dict name -> tensor with the checkpoint's names.

The design in short.  Sublayers come in sequence and read the residual x itself; a sublayer's result r is multiplied by a learned
gate and the sum is normed afterwards:  x <- LN(alpha x + sigmoid(R x + c) * r).  The token mixer reads a blend of x with the
previous token's x.  Mixers: retention (linear attention with one fixed decay per head) or latent attention (queries, keys and
values come out of low-rank latents, one rotated key part shared by all heads, a learned sink in the soft-max denominator, a
sigmoid gate per head).  Feed-forward: experts picked by a table indexed with the token id, plus a shared expert.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ---- norms -----------------------------------------------------------------------------------------------------------------------
def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(mean of squared deviations + eps) * w + b over the last dimension"""
    mu = x.mean(-1, keepdim=True)
    dev = x - mu
    return dev / torch.sqrt((dev * dev).mean(-1, keepdim=True) + eps) * w + b


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension"""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# ---- token shift -----------------------------------------------------------------------------------------------------------------
def token_shift(h: torch.Tensor, mu: torch.Tensor) -> torch.Tensor:
    """h [T, W] -> h_t + (h_(t-1) - h_t) * mu, with h_(-1) = 0; the previous row is taken before the blend"""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    return h + (prev - h) * mu


# ---- rotary positions --------------------------------------------------------------------------------------------------------------
def rotary_frequencies(rot: dict):
    """(frequency of every pair [dims / 2], factor on cos and sin)"""
    dims, base = rot["dims"], rot["base"]
    freq = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    amp = 1.0
    sc = rot.get("scaling")
    if sc:
        where = lambda turns: dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(where(sc["fast"])), 0)
        hi = min(math.ceil(where(sc["slow"])), dims - 1)
        for i in range(dims // 2):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            freq[i] = freq[i] / sc["factor"] * ramp + freq[i] * (1.0 - ramp)
        amp = 0.1 * math.log(sc["factor"]) + 1.0
    return freq, amp


def rotate(x: torch.Tensor, rot: Optional[dict], layout: str) -> torch.Tensor:
    """x [T, heads, D]; the first rot.dims dimensions of every head turn with the position, the rest passes.
    layout "half": dimension i pairs with i + dims / 2; "interleaved": 2i with 2i + 1"""
    if not rot:
        return x
    freq, amp = rotary_frequencies(rot)
    half = rot["dims"] // 2
    out = x.clone()
    for t in range(x.shape[0]):
        for i, f in enumerate(freq):
            a = t * f
            c, s = math.cos(a) * amp, math.sin(a) * amp
            iu, iv = (i, i + half) if layout == "half" else (2 * i, 2 * i + 1)
            u, v = x[t, :, iu], x[t, :, iv]
            out[t, :, iu] = u * c - v * s
            out[t, :, iv] = v * c + u * s
    return out


# ---- retention ---------------------------------------------------------------------------------------------------------------------
def retention_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: List[float]) -> torch.Tensor:
    """q, k [T, H, D], v [T, H, V]: S_t = decay_h S_(t-1) + k_t v_t^T (S_(-1) = 0), o_t = S_t^T q_t; no soft-max, no denominator"""
    T, H, D = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        S = torch.zeros(D, v.shape[2], dtype=q.dtype)
        for t in range(T):
            S = decay[h] * S + torch.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return out


def retention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, V)
    q, k = rotate(q, m.get("rot"), "half"), rotate(k, m.get("rot"), "half")
    k = k * D ** -0.5
    o = unit_rms(retention_scan(q, k, v, m["decay"]), eps).reshape(T, H * V)
    g = h @ w[p + "g"].T
    return (o * g * torch.sigmoid(g)) @ w[p + "o"].T


# ---- latent attention ----------------------------------------------------------------------------------------------------------------
def sink_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, sink: torch.Tensor) -> torch.Tensor:
    """q, k [T, H, D], v [T, H, V]; causal; the denominator of head h also holds exp(sink_h), which has no value"""
    T, H, _ = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for i in range(T):
        for h in range(H):
            s = (k[:i + 1, h] @ q[i, h]) * scale
            mx = max(float(s.max()), float(sink[h]))
            e = torch.exp(s - mx)
            out[i, h] = (e[:, None] * v[:i + 1, h]).sum(0) / (e.sum() + math.exp(float(sink[h]) - mx))
    return out


def latent_attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, Rd, V, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = unit_rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(T, H, D + Rd)
    kv = h @ w[p + "dkv"].T
    c = unit_rms(kv[:, :R], eps) * w[p + "dkv.norm"]
    kr = rotate(kv[:, None, R:], m.get("rot"), "interleaved")                 # [T, 1, Rd], one for all heads
    qr = rotate(q[:, :, D:], m.get("rot"), "interleaved")
    kn = (c @ w[p + "uk"].T).view(T, H, D)
    val = (c @ w[p + "uv"].T).view(T, H, V)
    qq = torch.cat([q[:, :, :D], qr], -1)
    kk = torch.cat([kn, kr.expand(T, H, Rd)], -1)
    o = sink_softmax_attention(qq, kk, val, m["scale"], w[p + "sink"])
    gate = torch.sigmoid(h @ w[p + "g"].T)                                       # [T, H]
    return (o * gate[:, :, None]).reshape(T, H * V) @ w[p + "o"].T


# ---- feed-forward ----------------------------------------------------------------------------------------------------------------------
def expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def table_experts(h: torch.Tensor, tokens: List[int], w: Dict[str, torch.Tensor], p: str, f: dict) -> torch.Tensor:
    """every token's experts come from row `token id` of the table, each weighted 1 / top; a shared expert is added"""
    top = f["router"]["top"]
    out = torch.zeros_like(h)
    for t, tok in enumerate(tokens):
        for j in range(top):
            e = int(w[p + "table"][tok, j])
            out[t] += expert(h[t:t + 1], w, p + f"e{e}.", f["expert"]["limit"])[0] / top
    if f.get("shared"):
        out = out + expert(h, w, p + "shared.", f["shared"]["limit"])
    return out


# ---- the model ---------------------------------------------------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None, dtype=torch.float64) -> torch.Tensor:
    """logits [T, vocab] of one sequence; layers_out collects the residual after every layer.  dtype float32 shows how far plain 32-bit
    rounding alone moves the result of a configuration (some are ill-conditioned: a unit norm over a single value, for instance)"""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = w["embed"][torch.tensor(tokens)]
    for i, lay in enumerate(cfg["layers"]):
        p = f"l{lay.get('weights_of', i)}."
        hs = token_shift(x, w[p + "shift"])
        if lay["type"] == "retention":
            r = retention_mixer(hs, w, p + "mix.", lay["mixer"], eps)
        elif lay["type"] == "latent_attention":
            r = latent_attention_mixer(hs, w, p + "mix.", lay["mixer"], eps)
        else:
            raise ValueError(lay["type"])
        r = r * torch.sigmoid(x @ w[p + "rg1"].T + w[p + "rg1.b"])
        x = layer_norm(alpha * x + r, w[p + "norm1"], w[p + "norm1.b"], eps)
        if lay.get("mlp"):
            r = table_experts(x, tokens, w, p + "mlp.", lay["mlp"])
            r = r * torch.sigmoid(x @ w[p + "rg2"].T + w[p + "rg2.b"])
            x = layer_norm(alpha * x + r, w[p + "norm2"], w[p + "norm2.b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return x @ w["embed"].T


# ---- random models and checkpoints (test fixtures) -------------------------------------------------------------------------------------
def random_model(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """random bfloat16-representable weights with the checkpoint's names and shapes; layers with weights_of get none"""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    r = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc).bfloat16().float()
    P = {"embed": r(V, W, sc=1.0), "final.norm": 1 + r(W, sc=0.1), "final.norm.b": r(W, sc=0.1)}
    for i, lay in enumerate(cfg["layers"]):
        if lay.get("weights_of") is not None:
            continue
        m, p = lay["mixer"], f"l{i}."
        subs = ("1", "2") if lay.get("mlp") else ("1",)
        for q in subs:
            P[p + "norm" + q], P[p + "norm" + q + ".b"] = 1 + r(W, sc=0.1), r(W, sc=0.1)
            P[p + "rg" + q], P[p + "rg" + q + ".b"] = r(W, W, sc=W ** -0.5), r(W, sc=0.5)
        P[p + "shift"] = torch.rand(W, generator=g).bfloat16().float()
        H = m["heads"]
        if lay["type"] == "retention":
            D, Vd = m["dim"], m["vdim"]
            P[p + "mix.q"], P[p + "mix.k"] = r(H * D, W, sc=2.0 * W ** -0.5), r(H * D, W, sc=2.0 * W ** -0.5)
            P[p + "mix.v"], P[p + "mix.g"] = r(H * Vd, W, sc=W ** -0.5), r(H * Vd, W, sc=W ** -0.5)
            P[p + "mix.o"] = r(W, H * Vd, sc=2.0 * (H * Vd) ** -0.5)
        else:
            D, Rd, Vd, R, Rq = m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            P[p + "mix.dq"], P[p + "mix.dq.norm"] = r(Rq, W, sc=W ** -0.5), 1 + r(Rq, sc=0.1)
            P[p + "mix.uq"] = r(H * (D + Rd), Rq, sc=2.0 * Rq ** -0.5)
            P[p + "mix.dkv"], P[p + "mix.dkv.norm"] = r(R + Rd, W, sc=W ** -0.5), 1 + r(R, sc=0.1)
            P[p + "mix.uk"], P[p + "mix.uv"] = r(H * D, R, sc=2.0 * R ** -0.5), r(H * Vd, R, sc=R ** -0.5)
            P[p + "mix.sink"] = r(H, sc=1.5)
            P[p + "mix.g"] = r(H, W, sc=W ** -0.5)
            P[p + "mix.o"] = r(W, H * Vd, sc=2.0 * (H * Vd) ** -0.5)
        mlp = lay.get("mlp")
        if mlp:
            E, top, ff = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
            for e in range(E):
                P[p + f"mlp.e{e}.gate"], P[p + f"mlp.e{e}.up"] = r(ff, W, sc=2.0 * W ** -0.5), r(ff, W, sc=2.0 * W ** -0.5)
                P[p + f"mlp.e{e}.down"] = r(W, ff, sc=2.0 * ff ** -0.5)
            P[p + "mlp.table"] = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(V)]).to(torch.int32)
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                P[p + "mlp.shared.gate"], P[p + "mlp.shared.up"] = r(sf, W, sc=2.0 * W ** -0.5), r(sf, W, sc=2.0 * W ** -0.5)
                P[p + "mlp.shared.down"] = r(W, sf, sc=2.0 * sf ** -0.5)
    return {k: (v.bfloat16().float() if v.is_floating_point() else v) for k, v in P.items()}      # the checkpoint holds bfloat16: what is not representable is rounded here


def write_checkpoint(folder: str, cfg: dict, P: Dict[str, torch.Tensor]) -> None:
    """config.json + model.safetensors (bfloat16, integer tables int32), written with the file format's own rules"""
    import json
    import os
    import struct

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    head, blobs, off = {}, [], 0
    for k, v in P.items():
        if v.is_floating_point():
            b, dt = v.bfloat16().contiguous().view(torch.uint8).numpy().tobytes(), "BF16"
        else:
            b, dt = v.to(torch.int32).contiguous().numpy().tobytes(), "I32"
        head[k] = {"dtype": dt, "shape": list(v.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(head).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
