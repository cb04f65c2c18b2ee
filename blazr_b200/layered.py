"""Layer-list models: a model is a list of layers, each one token mixer (attention over the paged KV pool, or a state-space
recurrence with per-slot state, retention, or latent attention) plus an optional feed-forward (dense or a mixture of experts),
wrapped in the pieces a design switches on.  Three layouts of the residual path exist:
  "streams": sublayers in sequence over several residual streams with learned mixing, grouped RMS norms and a short
             carried-state convolution in front of every sublayer (blazr_b200/fenorax.py);
  "depth":   parallel layers (mixer and feed-forward read the same input through two layer norms), one residual stream whose
             layer inputs are learned averages over the results of all earlier layers (blazr_b200/gemosun.py);
  "post":    sublayers in sequence that read the residual itself; a sublayer's result is multiplied by a learned sigmoid gate of the
             residual and the layer norm (weight and bias) comes after the sum, x <- LN(alpha x + gate * result); the mixer reads a
             blend of the residual with the previous token's (token shift, carried per sequence) (blazr_b200/teselix.py);
  "out_norm": sublayers in sequence that read the residual itself; the RMS norm sits on the sublayer's OUTPUT, x <- x + norm(sublayer(x));
             a mixer may be two branches side by side (an attention beside an element-wise gated recurrence) whose results are
             summed with fixed scales or after a norm of their own; a hashed bigram table may join the embedding and the logits
             may pass a soft cap (blazr_b200/pafelorn.py).
The mechanisms are parameterised (window / chunk / pooled-block size, score scale, unit-norm epsilon, rotary table, gate, state
size, activation kind, router groups, ...) so that another design can list them in another combination; a design is a function
config.json -> LayeredConfig.

One step function serves prefill, decode and mixed steps: `LayeredModel.forward(step)` takes a flat batch of tokens (prompt
portions beside single decoded tokens, blazr_b200/batch.py: build_step) and runs every layer once over all of them.  All math
runs in libb200seq kernels (blazr_b200/seqops.py); PyTorch holds the buffers.  What must be 32-bit is 32-bit in both modes:
the residual streams, norms, scores and soft-max, recurrent state, step sizes and decays, the KV pool.  `dtype` only selects
the activation type fed to the linear layers (bfloat16: tensor-core tiles; float32: exact fma tiles).

The decode-only step of a fixed batch size is captured into a CUDA graph (reference src/engine/cuda_graphs.rs:101-130).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch

from . import seqops
from .batch import StepArrays


# ---- specs -----------------------------------------------------------------------------------------------------------------
@dataclass
class RotarySpec:
    """rotary positions on the first `dims` dimensions of every q / k head, pairs (2i, 2i + 1); frequency base^(-2i / dims).
    yarn = (factor, original, fast, slow): frequencies whose wavelength fits `original` positions fewer than `slow` times are divided by
    `factor`, those that fit more than `fast` times stay, with a linear ramp over the pair index between; cos and sin are scaled
    by 0.1 ln(factor) + 1."""
    dims: int
    base: float
    yarn: Optional[tuple] = None
    layout: str = "interleaved"   # "interleaved": pairs (2i, 2i + 1); "half": pairs (i, i + dims / 2)
    linear: float = 1.0           # every frequency is divided by this
    # (factor, low, high, original): with wavelength l = 2 pi / f a frequency stays where l < original / high, is divided by factor where
    # l > original / low, and in between is (1 - s) f / factor + s f with s = (original / l - low) / (high - low)
    bands: Optional[tuple] = None

    def table(self):
        """(frequencies float32 [dims / 2], scale of cos and sin)"""
        import math
        i = np.arange(self.dims // 2, dtype=np.float64)
        f = self.base ** (-2.0 * i / self.dims)
        mscale = 1.0
        if self.yarn is not None:
            factor, original, fast, slow = self.yarn
            at = lambda turns: self.dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))
            lo, hi = max(math.floor(at(fast)), 0), min(math.ceil(at(slow)), self.dims - 1)
            ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / factor * ramp + f * (1.0 - ramp)
            mscale = 0.1 * math.log(factor) + 1.0
        if self.bands is not None:
            factor, low, high, original = self.bands
            wl = 2.0 * math.pi / f
            sm = (original / wl - low) / (high - low)
            f = np.where(wl < original / high, f, np.where(wl > original / low, f / factor, (1.0 - sm) * f / factor + sm * f))
        if self.linear != 1.0:
            f = f / self.linear
        return f.astype(np.float32), float(mscale)


@dataclass
class AttentionSpec:
    heads: int
    kv_heads: int
    dim: int                 # per-head query / key size
    vdim: int                # per-head value size
    scale: float
    chunk: int = 0           # > 0: a query sees only keys of its own chunk of this many positions (counted from position 0)
    window: int = 0          # > 0: a query sees only the last `window` positions
    qk_unit_norm: bool = True
    gated: bool = True       # one sigmoid gate per head on the output
    pool: int = 0            # > 0 (with window): blocks of `pool` positions wholly before the window are seen through their mean key / value
    values_from_keys: bool = False   # no value projection: v = k as projected (before norm and rotation)
    rot: Optional[RotarySpec] = None
    # ---- layout "out_norm" -------------------------------------------------------------------------------------------------------------
    qk_norm: str = "none"    # weighted RMS norm of q and k before rotation: "head" (per head, one weight [dim] for all heads) | "full" (over the whole projection)
    bias: bool = False       # q, k, v projections have biases
    out_bias: bool = False   # so has the output projection
    softcap: float = 0.0     # > 0: score <- softcap * tanh(score / softcap)
    head_temp: bool = False  # one learned factor per head on the scores
    sink: bool = False       # one learned logit per head joins the soft-max denominator (no key, no value)
    keep_first: int = 0      # with a window: the first positions of a sequence stay visible
    diff: Optional[float] = None   # differential attention: two maps per head over the same values, o = unit_rms(a1 - lambda a2) * (1 - diff)
    gate_elem: bool = False  # with gated: the sigmoid gate has one logit per output element (heads * vdim) instead of one per head
    kv_from: Optional[int] = None  # the keys and values are those of this (earlier) layer's cache; no k / v tensors of its own


@dataclass
class SsmSpec:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int                # taps of the convolution over x | B | C


@dataclass
class RetentionSpec:
    """linear attention with one fixed decay per head, no soft-max and no denominator: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t;
    rotary positions on q and k, k times dim^(-1/2), every head's o divided by its root mean square, times silu(gate), then the output projection"""
    heads: int
    dim: int                 # per-head query / key size
    vdim: int                # per-head value size
    decay: List[float] = field(default_factory=list)
    rot: Optional[RotarySpec] = None


@dataclass
class LatentAttentionSpec:
    """attention whose queries, keys and values come out of low-rank latents: c_q = rms_norm(W_dq h), q = W_uq c_q laid out per head as
    [dim unrotated | rot_dim rotated]; W_dkv h = [kv_rank latent (rms-normed: c) | rot_dim rotated key part shared by all heads]; per head the
    unrotated key is W_uk c and the value W_uv c.  Only c and the rotated key part are cached.  Causal soft-max over all earlier positions with
    an optional learned sink per head in the denominator and an optional sigmoid gate per head on the output."""
    heads: int
    dim: int                 # unrotated query / key dimensions per head
    rot_dim: int             # rotated dimensions per head
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: Optional[RotarySpec] = None
    sink: bool = True
    gated: bool = True


@dataclass
class MinGruSpec:
    """element-wise gated recurrence whose gates read only the current token: z = sigmoid(W_z h + b), u = W_x h + b, candidate u + 1/2 (u >= 0) or
    sigmoid(u); S_t = (1 - z) S_(t-1) + z candidate; output W_o (S_t * silu(W_g h)); f32 state per sequence"""
    width: int


@dataclass
class RgLruSpec:
    """recurrent block with a real-gated linear recurrent unit: y = gelu_tanh(W_y h + b), u = causal_conv(W_x h + b); per block of width / blocks
    channels r = sigmoid(A_r u + b), i = sigmoid(A_i u + b); a = exp(-decay * r * softplus(lam)); S_t = a S_(t-1) + sqrt(1 - a^2) i u;
    output W_o (S_t * y); f32 state and the last conv - 1 convolution inputs per sequence"""
    width: int
    blocks: int
    conv: int
    decay: float = 8.0


@dataclass
class TwoBranchSpec:
    """an attention (left) and a recurrence (right) read the same input; result = left_scale * left + right_scale * right, each branch first
    RMS-normed over the model width with a weight of its own when branch_norm"""
    left: AttentionSpec
    right: object            # MinGruSpec | RgLruSpec
    left_scale: float = 1.0
    right_scale: float = 1.0
    branch_norm: bool = False


@dataclass
class DenseFfSpec:
    ff: int
    limit: float = 0.0
    alpha: float = 1.702     # gate activation g * sigmoid(alpha * g)
    up_shift: float = 1.0    # (up + up_shift)
    # "swish_clamp": min(g, limit) * sigmoid(alpha * g) * (clamp(up) + up_shift); "gelu_tanh": gelu_tanh(g) * up;
    # "polynorm" (no gate projection): c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 with z = W_up h and N the division by the row's root mean square
    act: str = "swish_clamp"


@dataclass
class MoeFfSpec:
    """`top` of `experts` small feed-forwards per token - down(act(up h)), or with a gate branch down(act(gate h, up h)) - plus optionally a
    shared expert of the same form for every token.  router "sigmoid": the choice falls by sigmoid router scores among the experts of the
    `keep` best of `groups` groups of neighbours, weighted by their scores normalised over the chosen, the shared expert times a sigmoid
    token gate.  router "table": a table indexed by the token id names the experts, each weighted 1 / top, the shared expert is added as it is."""
    experts: int
    top: int
    ff: int
    groups: int = 1
    keep: int = 1
    act: str = "relu2"       # a plain kind: down(act(up h)); a gated kind ("swish_clamp"): down(act(gate h, up h)) with limit / alpha / up_shift
    shared_ff: int = 0       # 0: no shared expert
    shared_gate: bool = True
    # "sigmoid": learned router as above; "table": no router, a table [vocab, top] indexed by the token id names the experts, each weighted 1 / top;
    # "softmax": scores = soft-max over all router outputs, the choice adds a learned correction per output, the weights are the chosen scores normalised
    router: str = "sigmoid"
    identity: int = 0        # router "softmax": this many router outputs behind the experts' are identity experts (output = input, no tensors)
    correction: bool = False # router "softmax": tensor "correction" [experts + identity] joins the choice
    limit: float = 0.0
    alpha: float = 1.702
    up_shift: float = 1.0
    shared_limit: float = 0.0


@dataclass
class LayerSpec:
    kind: str                # "attention" | "ssm" | "retention" | "latent_attention" | "two_branch"
    mixer: object
    ff: Optional[object]     # DenseFfSpec | MoeFfSpec | None
    weights_of: Optional[int] = None   # layout "post": the layer has no tensors of its own and uses those of this (earlier) layer, with its own cache / state


@dataclass
class LayeredConfig:
    name: str
    vocab: int
    width: int
    streams: int
    norm_groups: int
    eps: float
    canon_taps: int          # taps of the convolution in front of every sublayer
    embed_scale: float
    layers: List[LayerSpec] = field(default_factory=list)
    layout: str = "streams"  # "streams" | "depth" (see the module text)
    tied_head: bool = True   # the output projection is the embedding table; False: a tensor "head"
    depth_average: bool = True   # layout "depth": layer i has weights "l<i>.dwa" [i + 2] over the embedding and the results of layers 0..i
    post_alpha: float = 1.0      # layout "post": weight of the residual in the sum that is normed
    bigram: Optional[tuple] = None   # layout "out_norm": (buckets, mul_prev, mul_cur) of the hashed bigram table "bigram" [buckets + 1, width]
    logit_softcap: float = 0.0       # > 0: logits <- cap * tanh(logits / cap)


class _Workspace:
    """device buffers of one step capacity (addresses stay put: a step of fixed shape can be graph-captured)"""

    def __init__(self, model: "LayeredModel", cap: int):
        cfg, dev = model.cfg, model.dev
        f32 = dict(dtype=torch.float32, device=dev)
        act = dict(dtype=model.act_dtype, device=dev)
        self.cap = cap
        W = cfg.width
        self.X = torch.empty((cap, cfg.streams, W), **f32)
        self.h = torch.empty((cap, W), **f32)
        self.a = torch.empty((cap, W), **act)
        self.y = torch.empty((cap, W), **f32)
        self.proj = torch.empty((cap, model.max_proj), **f32)
        self.xbc = torch.empty((cap, max(1, model.max_xbc)), **f32)
        self.inner_f = torch.empty((cap, max(1, model.max_inner)), **f32)
        self.inner_a = torch.empty((cap, max(1, model.max_inner)), **act)
        self.fin = torch.empty((cap, W), **act)
        self.logits = torch.empty((cap, cfg.vocab), **f32)
        if cfg.layout == "depth":       # results of the embedding and of every layer but the last (the depth average reads them), second branch
            self.hist = torch.empty((max(1, len(cfg.layers)), cap, W), **f32)
            self.xbuf = torch.empty((cap, W), **f32)
            self.a2 = torch.empty((cap, W), **act)
            self.y2 = torch.empty((cap, W), **f32)
            # the feed-forward branch runs beside the mixer on a second stream: it keeps its own intermediates
            self.ff_inner = torch.empty((cap, max(1, model.max_ff_inner)), **act)
            self.ff_proj = torch.empty((cap, max(1, model.max_ff_proj)), **f32)
        if cfg.layout == "post":        # shifted activations, gate logits, buffers of the latent-attention mixer, the shared expert's intermediates
            self.a2 = torch.empty((cap, W), **act)
            self.zg = torch.empty((cap, W), **f32)
            self.q = torch.empty((cap, max(1, model.max_q)), **f32)
            self.Qp = torch.empty((cap, max(1, model.max_qp)), **f32)
            self.qn = torch.empty((cap, max(1, model.max_qn)), **act)
            self.oup = torch.empty((cap, max(1, model.max_inner)), **act)
            self.ff_inner = torch.empty((cap, max(1, model.max_ff_inner)), **act)
            self.ff_proj = torch.empty((cap, max(1, model.max_ff_proj)), **f32)
        if cfg.layout == "out_norm":    # second branch of a two-branch mixer, the recurrences' intermediates, the feed-forward's own buffers
            self.y2 = torch.empty((cap, W), **f32)
            self.inner_b = torch.empty((cap, max(1, model.max_rinner)), **act)
            self.conv_a = torch.empty((cap, max(1, model.max_xbc)), **act)
            self.gates = torch.empty((cap, 2 * max(1, model.max_xbc)), **f32)
            self.ff_inner = torch.empty((cap, max(1, model.max_ff_inner)), **act)
            self.ff_proj = torch.empty((cap, max(1, model.max_ff_proj)), **f32)
        mo = model.moe_dims
        if mo is not None:              # mixture of experts: router logits, choices, sort, per-pair intermediates
            E1, top, F = mo
            i32 = dict(dtype=torch.int32, device=dev)
            self.moe_z = torch.empty((cap, E1), **f32)
            self.moe_ids = torch.empty((cap * top,), **i32)
            self.moe_wts = torch.empty((cap * top,), **f32)
            self.moe_cnt = torch.zeros((E1,), **i32)
            self.moe_off = torch.zeros((E1 + 1,), **i32)
            self.moe_order = torch.empty((cap * top,), **i32)
            self.moe_slot = torch.empty((cap * top,), **i32)
            self.moe_act = torch.empty((cap * top, F), **act)
            self.moe_ys = torch.empty((cap * top, W), **f32)
            self.moe_sh = torch.empty((cap, W), **f32)
            self.moe_xs = torch.empty((cap * top, W), **act) if model.act_dtype == torch.bfloat16 else None   # tokens' rows in sorted pair order
            # table-routed layers choose (and sort) at the start of the step, each into buffers of its own
            self.route = {}
            for i, L in enumerate(model.layers):
                f = L["spec"].ff
                if isinstance(f, MoeFfSpec) and f.router == "table":
                    n = cap * f.top
                    self.route[i] = dict(ids=torch.empty(n, **i32), wts=torch.empty(n, **f32), cnt=torch.zeros(f.experts, **i32), off=torch.zeros(f.experts + 1, **i32),
                                         order=torch.empty(n, **i32), slot=torch.empty(n, **i32))
        self.scratch = torch.empty(max(1, model.scratch_floats(cap)), **f32)      # work area: segmented state-space scan, key-split attention
        self.next_ids = torch.empty((cap,), dtype=torch.int32, device=dev)
        # int32 step arrays in one buffer: ids | ent | pos | want | start | slot | pos0 | prev | block_table
        B, mb = model.max_seqs, model.max_blocks
        self.off = {}
        o = 0
        for k, n in (("ids", cap), ("ent", cap), ("pos", cap), ("want", cap), ("start", B + 1), ("slot", B), ("pos0", B), ("prev", B), ("bt", B * mb)):
            self.off[k] = (o, n)
            o += -(-n // 4) * 4
        self.meta = torch.zeros(o, dtype=torch.int32, device=dev)
        self.copied = None
        self.meta_host = torch.zeros(o, dtype=torch.int32).pin_memory() if dev.type == "cuda" else torch.zeros(o, dtype=torch.int32)

    def view(self, k: str) -> torch.Tensor:
        o, n = self.off[k]
        return self.meta[o:o + n]


class LayeredModel:
    """weights + per-layer cache / state + the step function"""

    def __init__(self, cfg: LayeredConfig, tensors, device, dtype: str = "bfloat16"):
        """tensors: name -> torch CPU tensor (callable or mapping with the checkpoint's names)"""
        if dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype {dtype}: bfloat16 or float32")
        self.cfg, self.dev, self.dtype = cfg, torch.device(device), dtype
        self.act_dtype = torch.bfloat16 if dtype == "bfloat16" else torch.float32
        get = tensors if callable(tensors) else tensors.__getitem__
        dev = self.dev
        S, W = cfg.streams, cfg.width
        if S > 8 or cfg.canon_taps > 8:
            raise ValueError("at most 8 residual streams and 8 convolution taps")

        def lin(*names):   # linear weights stay bfloat16; several projections of one input are stacked along N (one launch)
            parts = []
            for n in names:
                t = get(n)
                if t.dtype != torch.bfloat16:
                    if dtype == "float32" and t.dtype in (torch.float32, torch.float64) and not torch.equal(t.bfloat16().to(t.dtype), t):
                        raise ValueError(f"{n}: float32 mode needs weights that are exact in bfloat16")
                    t = t.to(torch.bfloat16)
                parts.append(t)
            return torch.cat(parts, 0).contiguous().to(dev)

        def vec(name):
            return get(name).to(torch.float32).contiguous().to(dev)

        def hc(pre):    # (in [S], post = out [S] | mix [S, S])
            return vec(pre + "in"), torch.cat([get(pre + "out").float().reshape(-1), get(pre + "mix").float().reshape(-1)]).contiguous().to(dev)

        if cfg.layout not in ("streams", "depth", "post", "out_norm"):
            raise ValueError(f"unknown residual layout {cfg.layout}")
        depth, post, outn = cfg.layout == "depth", cfg.layout == "post", cfg.layout == "out_norm"
        if (depth or post or outn) and (S != 1 or cfg.canon_taps > 1):
            raise ValueError("the depth-averaged and post-norm layouts have one residual stream and no carried convolution")
        self.embed = lin("embed")
        self.head = self.embed if cfg.tied_head else lin("head")
        self.final_norm = vec("final.norm")
        self.final_bias = vec("final.norm.b") if post else None
        if tuple(self.embed.shape) != (cfg.vocab, W) or tuple(self.head.shape) != (cfg.vocab, W) or self.final_norm.numel() != W:
            raise ValueError("embedding / head / final norm shapes do not fit the configuration")
        self.ones_in = torch.ones(S, dtype=torch.float32, device=dev)
        self.bigram = None
        if cfg.bigram is not None:
            if not outn:
                raise ValueError("the bigram table is wired into the out_norm layout")
            self.bigram = lin("bigram")
            if tuple(self.bigram.shape) != (int(cfg.bigram[0]) + 1, W) or int(cfg.bigram[0]) < 1:
                raise ValueError("the bigram table has buckets + 1 rows of the model width")
        self.layers: List[Dict[str, object]] = []
        self.max_rinner = 1      # out_norm layout: widest recurrent branch
        self.max_proj = self.max_xbc = self.max_inner = 1
        self.max_ff_inner = self.max_ff_proj = 1      # depth layout: sizes of the feed-forward branch's own intermediates
        self.moe_dims = None      # (experts + 1, top, expert ff): largest over the layers
        self.max_q = self.max_qp = self.max_qn = 1      # latent attention: query rows, latent-space query rows, unrotated query parts
        self.max_ctx_r = self.max_ctx_kv = 0            # latent attention: latent size, per-head keys | values of one position
        self.weight_bytes = self.embed.numel() * 2 + (0 if cfg.tied_head else self.head.numel() * 2) + (self.bigram.numel() * 2 if self.bigram is not None else 0)
        for i, ls in enumerate(cfg.layers):
            if post:
                self.layers.append(self._post_layer(i, ls, lin, vec, get))
                continue
            if outn:
                self.layers.append(self._out_layer(i, ls, lin, vec, get))
                continue
            L: Dict[str, object] = {"spec": ls}
            p = f"l{i}."
            L["norm1"] = vec(p + "norm1")
            if depth:
                if L["norm1"].numel() != W:
                    raise ValueError(f"layer {i}: norm weight does not fit the width")
                L["dwa"] = vec(p + "dwa") if cfg.depth_average else None      # None: the plain residual sum goes on
                if L["dwa"] is not None and L["dwa"].numel() != i + 2:
                    raise ValueError(f"layer {i}: {i + 2} depth weights expected")
            else:
                L["canon1"] = vec(p + "canon1")
                L["hc1_in"], L["hc1_post"] = hc(p + "hc1.")
            m = ls.mixer
            if ls.kind == "attention":
                names = [p + "mix.q", p + "mix.k"] + ([] if m.values_from_keys else [p + "mix.v"]) + ([p + "mix.g"] if m.gated else [])
                L["w_in"] = lin(*names)
                L["w_o"] = lin(p + "mix.o")
                if m.values_from_keys and m.vdim != m.dim:
                    raise ValueError(f"layer {i}: values taken from the keys need vdim == dim")
                if m.pool > 0 and m.window < 1:
                    raise ValueError(f"layer {i}: pooled blocks need a window")
                rot_freq, rot_scale = None, 1.0
                if m.rot is not None:
                    if m.rot.dims < 2 or m.rot.dims % 2 or m.rot.dims > m.dim:
                        raise ValueError(f"layer {i}: rotary dimensions must be even and at most the head size")
                    fr, rot_scale = m.rot.table()
                    rot_freq = torch.from_numpy(fr).to(dev)
                L["rot_freq"] = rot_freq
                L["desc"] = seqops.attn_desc(m.heads, m.kv_heads, m.dim, m.vdim, m.scale, values_from_keys=m.values_from_keys, gated=m.gated, chunk=m.chunk,
                                             window=m.window, pool=m.pool, qk_eps=cfg.eps if m.qk_unit_norm else -1.0, rot_freq=rot_freq, rot_scale=rot_scale)
                n_in = L["desc"].width
                if tuple(L["w_in"].shape) != (n_in, W) or tuple(L["w_o"].shape) != (W, m.heads * m.vdim):
                    raise ValueError(f"layer {i}: attention tensor shapes do not fit the configuration")
                self.max_inner = max(self.max_inner, m.heads * m.vdim)
            elif ls.kind == "ssm":
                L["w_in"] = lin(p + "mix.in")
                L["w_o"] = lin(p + "mix.o")
                L["conv_w"], L["conv_b"] = vec(p + "mix.conv"), vec(p + "mix.conv.b")
                L["dt_bias"], L["A_log"], L["D"], L["mnorm"] = vec(p + "mix.dt_bias"), vec(p + "mix.A_log"), vec(p + "mix.D"), vec(p + "mix.norm")
                inner, gn = m.heads * m.vdim, m.groups * m.state
                if tuple(L["w_in"].shape) != (2 * inner + 2 * gn + m.heads, W) or tuple(L["conv_w"].shape) != (inner + 2 * gn, m.conv):
                    raise ValueError(f"layer {i}: state-space tensor shapes do not fit the configuration")
                self.max_inner = max(self.max_inner, inner)
                self.max_xbc = max(self.max_xbc, inner + 2 * gn)
            else:
                raise ValueError(f"layer {i}: unknown mixer kind {ls.kind}")
            self.max_proj = max(self.max_proj, L["w_in"].shape[0])
            self.weight_bytes += (L["w_in"].numel() + L["w_o"].numel()) * 2
            if isinstance(ls.ff, MoeFfSpec):
                f = ls.ff
                if f.act not in ("relu2",) or seqops.ACT_KINDS[f.act] in seqops.ACT_GATED or f.router != "sigmoid":
                    raise ValueError(f"layer {i}: expert activation {f.act} / router {f.router} is not supported in this layout")
                if f.top > f.experts or (f.groups > 1 and (f.experts % f.groups or not 1 <= f.keep <= f.groups or f.keep * (f.experts // f.groups) < f.top)):
                    raise ValueError(f"layer {i}: router groups / top do not fit the expert count")
                L["norm2"] = vec(p + "norm2")
                router = [p + "mlp.router"] + ([p + "mlp.shared.sg"] if f.shared_ff and f.shared_gate else [])
                L["w_router"] = lin(*router)          # the shared expert's token gate rides as one more row
                L["w_eup"] = torch.stack([lin(p + f"mlp.e{e}.up") for e in range(f.experts)]).contiguous()
                L["w_edown"] = torch.stack([lin(p + f"mlp.e{e}.down") for e in range(f.experts)]).contiguous()
                if tuple(L["w_router"].shape) != (len(router) - 1 + f.experts, W) or tuple(L["w_eup"].shape[1:]) != (f.ff, W) or tuple(L["w_edown"].shape[1:]) != (W, f.ff):
                    raise ValueError(f"layer {i}: router / expert tensor shapes do not fit the configuration")
                self.weight_bytes += (L["w_router"].numel() + L["w_eup"].numel() + L["w_edown"].numel()) * 2
                if f.shared_ff:
                    L["w_sup"], L["w_sdown"] = lin(p + "mlp.shared.up"), lin(p + "mlp.shared.down")
                    if tuple(L["w_sup"].shape) != (f.shared_ff, W) or tuple(L["w_sdown"].shape) != (W, f.shared_ff):
                        raise ValueError(f"layer {i}: shared expert tensor shapes do not fit the configuration")
                    self.weight_bytes += (L["w_sup"].numel() + L["w_sdown"].numel()) * 2
                    self.max_ff_inner = max(self.max_ff_inner, f.shared_ff)
                    self.max_ff_proj = max(self.max_ff_proj, f.shared_ff)
                md = self.moe_dims or (1, 1, 1)
                self.moe_dims = (max(md[0], f.experts + 1), max(md[1], f.top), max(md[2], f.ff))
                if not depth:
                    raise ValueError("mixture-of-experts feed-forwards are wired into the depth-averaged layout only")
            elif ls.ff is not None:
                L["norm2"] = vec(p + "norm2")
                if not depth:
                    L["canon2"] = vec(p + "canon2")
                    L["hc2_in"], L["hc2_post"] = hc(p + "hc2.")
                if ls.ff.act not in seqops.ACT_KINDS or seqops.ACT_KINDS[ls.ff.act] not in seqops.ACT_GATED:
                    raise ValueError(f"layer {i}: dense feed-forward activation {ls.ff.act} is not a gated kind")
                gu = lin(p + "mlp.gate", p + "mlp.up")          # stored with alternating rows (gate j, up j): the pair meets in one warp
                L["w_gu"] = gu.view(2, ls.ff.ff, W).transpose(0, 1).reshape(2 * ls.ff.ff, W).contiguous()
                L["w_down"] = lin(p + "mlp.down")
                if tuple(gu.shape) != (2 * ls.ff.ff, W) or tuple(L["w_down"].shape) != (W, ls.ff.ff):
                    raise ValueError(f"layer {i}: feed-forward tensor shapes do not fit the configuration")
                if depth:
                    self.max_ff_proj = max(self.max_ff_proj, 2 * ls.ff.ff)
                    self.max_ff_inner = max(self.max_ff_inner, ls.ff.ff)
                else:
                    self.max_proj = max(self.max_proj, 2 * ls.ff.ff)
                    self.max_inner = max(self.max_inner, ls.ff.ff)
                self.weight_bytes += (L["w_gu"].numel() + L["w_down"].numel()) * 2
            self.layers.append(L)
        self.max_seqs = self.max_blocks = self.block_size = 0
        self._ws: Dict[int, _Workspace] = {}
        self._graphs: Dict[int, object] = {}
        self.use_graphs = True
        self.overlap_branches = True     # depth layout: mixer and feed-forward of a layer on two streams
        self._side = self._side2 = None
        self._ctx_rows = 0       # steps with prompt portions: positions in the contexts of all entries (latent attention projects keys / values out of them)
        self._ctx_cap, self._ctx = 0, None

    # ---- layout "post": weights of one layer -------------------------------------------------------------------------------------------
    def _post_layer(self, i: int, ls: "LayerSpec", lin, vec, get) -> Dict[str, object]:
        cfg, dev, W = self.cfg, self.dev, self.cfg.width
        m, f = ls.mixer, ls.ff
        if ls.weights_of is not None:     # the tensors of an earlier layer; cache and state are this layer's own (allocate())
            j = ls.weights_of
            if not 0 <= j < i or cfg.layers[j].weights_of is not None:
                raise ValueError(f"layer {i}: weights_of must name an earlier layer that has tensors of its own")
            if cfg.layers[j].kind != ls.kind or cfg.layers[j].mixer != m or cfg.layers[j].ff != f:
                raise ValueError(f"layer {i}: a layer that shares weights has the sizes of the layer it shares them with")
            L = dict(self.layers[j])
            L["spec"] = ls
            self._post_sizes(L, ls)
            return L
        L: Dict[str, object] = {"spec": ls}
        p = f"l{i}."
        sub = (1, 2) if f is not None else (1,)
        for q in sub:
            L[f"norm{q}"], L[f"norm{q}_b"] = vec(p + f"norm{q}"), vec(p + f"norm{q}.b")
            L[f"rg{q}"], L[f"rg{q}_b"] = lin(p + f"rg{q}"), vec(p + f"rg{q}.b")
            if L[f"norm{q}"].numel() != W or L[f"norm{q}_b"].numel() != W or tuple(L[f"rg{q}"].shape) != (W, W) or L[f"rg{q}_b"].numel() != W:
                raise ValueError(f"layer {i}: norm / residual-gate tensor shapes do not fit the width")
            self.weight_bytes += L[f"rg{q}"].numel() * 2
        L["shift"] = vec(p + "shift")
        if L["shift"].numel() != W:
            raise ValueError(f"layer {i}: token-shift weight does not fit the width")

        def rotary(rot, size, what):
            if rot is None:
                return None, 1.0
            if rot.dims < 2 or rot.dims % 2 or rot.dims > size:
                raise ValueError(f"layer {i}: rotary dimensions must be even and at most {what}")
            fr, scale = rot.table()
            return torch.from_numpy(fr).to(dev), scale

        if ls.kind == "retention":
            import math
            H, D, V = m.heads, m.dim, m.vdim
            L["w_in"] = lin(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g")
            L["w_o"] = lin(p + "mix.o")
            if tuple(L["w_in"].shape) != (2 * H * D + 2 * H * V, W) or tuple(L["w_o"].shape) != (W, H * V) or len(m.decay) != H:
                raise ValueError(f"layer {i}: retention tensor shapes / decay list do not fit the configuration")
            if any(not 0.0 < float(d) <= 1.0 for d in m.decay):
                raise ValueError(f"layer {i}: decays lie in (0, 1]")
            L["decay"] = torch.tensor([[float(d) for d in m.decay], [math.log2(float(d)) for d in m.decay]], dtype=torch.float64).to(torch.float32).to(dev)
            L["rot_freq"], rot_scale = rotary(m.rot, D, "the key size")
            if m.rot is not None and m.rot.layout not in ("half", "interleaved"):
                raise ValueError(f"layer {i}: unknown rotary layout {m.rot.layout}")
            L["desc"] = seqops.retention_desc(H, D, V, L["decay"], cfg.eps, float(D) ** -0.5, rot_freq=L["rot_freq"],
                                              rot_half=m.rot is not None and m.rot.layout == "half", rot_scale=rot_scale)
        elif ls.kind == "latent_attention":
            H, Dn, Rd, V, R, Rq = m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank
            if m.rot is not None and (m.rot.dims != Rd or m.rot.layout != "interleaved"):
                raise ValueError(f"layer {i}: the rotated part turns as a whole, in interleaved pairs")
            if (m.rot is None) != (Rd == 0):
                raise ValueError(f"layer {i}: a rotated part needs rotary constants (and the other way round)")
            L["w_in"] = lin(*([p + "mix.dq", p + "mix.dkv"] + ([p + "mix.g"] if m.gated else [])))     # one projection of the shifted input: c_q | c, k_rot | gates
            L["dq_norm"], L["kv_norm"] = vec(p + "mix.dq.norm"), vec(p + "mix.dkv.norm")
            L["w_uq"], L["w_o"] = lin(p + "mix.uq"), lin(p + "mix.o")
            uk, uv = lin(p + "mix.uk"), lin(p + "mix.uv")
            if tuple(L["w_in"].shape) != (Rq + R + Rd + (H if m.gated else 0), W) or tuple(L["w_uq"].shape) != (H * (Dn + Rd), Rq) or tuple(uk.shape) != (H * Dn, R) \
                    or tuple(uv.shape) != (H * V, R) or tuple(L["w_o"].shape) != (W, H * V) or L["dq_norm"].numel() != Rq or L["kv_norm"].numel() != R:
                raise ValueError(f"layer {i}: latent-attention tensor shapes do not fit the configuration")
            L["w_ukT"] = uk.view(H, Dn, R).transpose(1, 2).contiguous()      # [H][R][Dn]: the query's way into the latent space
            L["w_uv"] = uv.view(H, V, R).contiguous()
            L["w_ukv"] = torch.cat([uk, uv], 0).contiguous()                 # steps of prompt portions: per-head keys | values out of the gathered latents
            L["sink"] = vec(p + "mix.sink") if m.sink else None
            if m.sink and L["sink"].numel() != H:
                raise ValueError(f"layer {i}: one sink per head expected")
            L["rot_freq"], L["rot_scale"] = rotary(m.rot, max(Rd, 2), "the rotated part")
            L["desc"] = seqops.latent_attn_desc(H, R, Rd, m.scale, gated=m.gated, sink=L["sink"])
            self.weight_bytes += (L["w_uq"].numel() + uk.numel() + uv.numel()) * 2
        else:
            raise ValueError(f"layer {i}: mixer kind {ls.kind} is not wired into the post-norm layout")
        self.weight_bytes += (L["w_in"].numel() + L["w_o"].numel()) * 2

        def gate_up(pre, ff):      # rows alternate (gate j, up j): the pair meets in one warp / neighbouring lanes
            gu = lin(pre + "gate", pre + "up")
            if tuple(gu.shape) != (2 * ff, W):
                raise ValueError(f"layer {i}: {pre}gate / up shapes do not fit the configuration")
            return gu.view(2, ff, W).transpose(0, 1).reshape(2 * ff, W).contiguous()

        if isinstance(f, MoeFfSpec):
            self._load_moe(L, i, f, lin, vec, get)
        elif f is not None:
            if f.act not in seqops.ACT_KINDS or seqops.ACT_KINDS[f.act] not in seqops.ACT_GATED:
                raise ValueError(f"layer {i}: dense feed-forward activation {f.act} is not a gated kind")
            L["w_gu"] = gate_up(p + "mlp.", f.ff)
            L["w_down"] = lin(p + "mlp.down")
            if tuple(L["w_down"].shape) != (W, f.ff):
                raise ValueError(f"layer {i}: feed-forward tensor shapes do not fit the configuration")
            self.weight_bytes += (L["w_gu"].numel() + L["w_down"].numel()) * 2
        self._post_sizes(L, ls)
        return L

    # ---- layout "out_norm": weights of one layer ------------------------------------------------------------------------------------------
    def _out_layer(self, i: int, ls: "LayerSpec", lin, vec, get) -> Dict[str, object]:
        """One stacked input projection per mixer: [q | k | v | gate] of the attention, then the recurrent branch's projections; the biases of the
        projections form one f32 vector indexed by the stacked row's columns (zero where a projection has none), added by the kernels that read the row."""
        import math
        cfg, dev, W = self.cfg, self.dev, self.cfg.width
        L: Dict[str, object] = {"spec": ls}
        p = f"l{i}."
        L["norm1"] = vec(p + "norm1")
        if L["norm1"].numel() != W:
            raise ValueError(f"layer {i}: norm weight does not fit the width")
        if ls.kind == "attention":
            att, right, ap = ls.mixer, None, p + "mix."
        elif ls.kind == "two_branch":
            att, right, ap = ls.mixer.left, ls.mixer.right, p + "mix.left."
        else:
            raise ValueError(f"layer {i}: mixer kind {ls.kind} is not wired into the out_norm layout")
        m = att
        H, G, D, V = m.heads, m.kv_heads, m.dim, m.vdim
        if H % G or m.values_from_keys or m.pool or m.chunk:
            raise ValueError(f"layer {i}: attention options that this layout does not wire (or heads not a multiple of kv_heads)")
        maps = 2 if m.diff is not None else 1
        shared = m.kv_from is not None
        if shared:
            j = m.kv_from
            src = cfg.layers[j] if 0 <= j < i else None
            sm = None if src is None else (src.mixer if src.kind == "attention" else src.mixer.left if src.kind == "two_branch" else None)
            if sm is None or sm.kv_from is not None or (sm.heads, sm.kv_heads, sm.dim, sm.vdim, sm.diff is None) != (H, G, D, V, m.diff is None):
                raise ValueError(f"layer {i}: kv_from must name an earlier attention layer with keys of its own and the same head counts and sizes")
        parts, biases = [], []

        def add(name, rows, bias, perm=None):
            t = get(name)
            if tuple(t.shape) != (rows, W):
                raise ValueError(f"layer {i}: {name} has shape {tuple(t.shape)}, expected {(rows, W)}")
            b = get(name + ".b").float().reshape(-1) if bias else torch.zeros(rows)
            if b.numel() != rows:
                raise ValueError(f"layer {i}: {name}.b does not fit")
            if perm is not None:
                t, b = perm(t), perm(b)
            parts.append(t.to(torch.bfloat16) if t.dtype != torch.bfloat16 else t)
            biases.append(b)

        # differential attention: the query rows come head by head as [map 1 | map 2]; they are reordered to [key group][map][head of the group] so
        # that the two maps are 2 H plain query heads over 2 G key heads (query head h' reads key head h' / (H / G)) that share G value heads
        R = H // G
        qperm = (lambda t: t.reshape(G, R, 2, D, *t.shape[1:]).transpose(1, 2).reshape(t.shape)) if maps == 2 else None
        add(ap + "q", H * maps * D, m.bias, qperm)
        if not shared:
            add(ap + "k", G * maps * D, m.bias)
            add(ap + "v", G * V, m.bias)
        if m.gated:
            add(ap + "g", H * V if m.gate_elem else H, False)
        n_att = sum(t.shape[0] for t in parts)
        rc = {}
        if isinstance(right, MinGruSpec):
            C = right.width
            for nm, b in (("z", True), ("x", True), ("g", False)):
                rc[nm] = sum(t.shape[0] for t in parts)
                add(p + "mix.right." + nm, C, b)
        elif isinstance(right, RgLruSpec):
            C = right.width
            if right.blocks < 1 or C % right.blocks or not 1 <= right.conv <= 8:
                raise ValueError(f"layer {i}: blocks must divide the recurrent width, 1..8 convolution taps")
            for nm in ("y", "x"):
                rc[nm] = sum(t.shape[0] for t in parts)
                add(p + "mix.right." + nm, C, True)
        elif right is not None:
            raise ValueError(f"layer {i}: unknown recurrent branch {type(right).__name__}")
        L["w_in"] = torch.cat(parts, 0).contiguous().to(dev)
        bias = torch.cat(biases).to(torch.float32)
        L["in_bias"] = bias.contiguous().to(dev) if bool((bias != 0).any()) else None
        L["w_o"] = lin(ap + "o")
        if tuple(L["w_o"].shape) != (W, H * V):
            raise ValueError(f"layer {i}: output projection shape does not fit")
        L["o_bias"] = vec(ap + "o.b") if m.out_bias else None
        self.weight_bytes += (L["w_in"].numel() + L["w_o"].numel()) * 2
        rot_freq, rot_scale = None, 1.0
        if m.rot is not None:
            if m.rot.dims < 2 or m.rot.dims % 2 or m.rot.dims > D or m.rot.layout not in ("half", "interleaved"):
                raise ValueError(f"layer {i}: rotary dimensions must be even and at most the head size, layout half or interleaved")
            fr, rot_scale = m.rot.table()
            rot_freq = torch.from_numpy(fr).to(dev)
        L["rot_freq"] = rot_freq
        if m.qk_norm not in ("none", "head", "full"):
            raise ValueError(f"layer {i}: unknown q / k norm {m.qk_norm}")
        L["q_norm_w"] = vec(ap + "q.norm") if m.qk_norm != "none" else None
        L["k_norm_w"] = vec(ap + "k.norm") if m.qk_norm != "none" and not shared else None
        nq, nk = (D, D) if m.qk_norm == "head" else (H * maps * D, G * maps * D)
        if L["q_norm_w"] is not None and (L["q_norm_w"].numel() != nq or (L["k_norm_w"] is not None and L["k_norm_w"].numel() != nk)):
            raise ValueError(f"layer {i}: q / k norm weights do not fit")
        if m.qk_norm == "full" and maps == 2:
            raise ValueError(f"layer {i}: a norm over the whole projection is not wired for differential attention")
        L["temp"] = vec(ap + "temp") if m.head_temp else None
        L["sink"] = vec(ap + "sink") if m.sink else None
        if (L["temp"] is not None and L["temp"].numel() != H) or (L["sink"] is not None and L["sink"].numel() != H) or (maps == 2 and (m.head_temp or m.sink)):
            raise ValueError(f"layer {i}: one temperature / sink per head (not with differential attention)")
        L["desc"] = seqops.attn_desc(H * maps, G * maps, D, V, m.scale, gated=m.gated, gate_elem=m.gate_elem, window=m.window,
                                     qk_eps=cfg.eps if (m.qk_norm != "none" or m.qk_unit_norm) else -1.0, rot_freq=rot_freq, rot_scale=rot_scale, sink=L["sink"],
                                     q_norm_w=L["q_norm_w"], k_norm_w=L["k_norm_w"], norm_full=m.qk_norm == "full", rot_half=m.rot is not None and m.rot.layout == "half",
                                     in_bias=L["in_bias"], kv_shared=shared, value_heads=G if maps == 2 else 0, softcap=m.softcap, head_scale=L["temp"],
                                     keep_first=m.keep_first if m.window > 0 else 0)
        if L["desc"].width != n_att:
            raise AssertionError("attention columns of the stacked projection")
        if maps == 2:
            for nm in ("lq1", "lk1", "lq2", "lk2"):
                if get(ap + nm).numel() != D:
                    raise ValueError(f"layer {i}: {nm} has the head size")
            f64 = lambda nm: get(ap + nm).to(torch.float64).reshape(-1)
            L["lambda"] = float(torch.exp((f64("lq1") * f64("lk1")).sum()) - torch.exp((f64("lq2") * f64("lk2")).sum())) + float(m.diff)
        self.max_inner = max(self.max_inner, H * V * maps)
        L["rcols"] = rc
        if isinstance(right, MinGruSpec):
            L["w_ro"] = lin(p + "mix.right.o")
        elif isinstance(right, RgLruSpec):
            C, nb = right.width, right.blocks
            bw = C // nb
            L["w_ro"] = lin(p + "mix.right.o")
            L["conv_w"], L["conv_b"] = vec(p + "mix.right.conv"), vec(p + "mix.right.conv.b")
            ra, ri = get(p + "mix.right.ra"), get(p + "mix.right.ri")
            if tuple(ra.shape) != (nb, bw, bw) or tuple(ri.shape) != (nb, bw, bw) or tuple(L["conv_w"].shape) != (C, right.conv) or L["conv_b"].numel() != C:
                raise ValueError(f"layer {i}: recurrent gate / convolution tensor shapes do not fit")
            L["w_gates"] = torch.cat([ra.to(torch.bfloat16), ri.to(torch.bfloat16)], 1).contiguous().to(dev)      # [blocks][r rows | i rows][bw]
            L["gate_bias"] = torch.cat([get(p + "mix.right.ra.b").float().reshape(nb, bw), get(p + "mix.right.ri.b").float().reshape(nb, bw)], 1).reshape(-1).contiguous().to(dev)
            lam = get(p + "mix.right.lam").to(torch.float64).reshape(-1)
            if lam.numel() != C:
                raise ValueError(f"layer {i}: lam has the recurrent width")
            L["sp_lam"] = torch.nn.functional.softplus(lam).to(torch.float32).contiguous().to(dev)
            L["x_bias"] = L["in_bias"][rc["x"]:rc["x"] + C] if L["in_bias"] is not None else None
            self.max_xbc = max(self.max_xbc, C)
            self.weight_bytes += L["w_gates"].numel() * 2
        if right is not None:
            if tuple(L["w_ro"].shape) != (W, right.width):
                raise ValueError(f"layer {i}: recurrent output projection shape does not fit")
            self.max_rinner = max(self.max_rinner, right.width)
            self.weight_bytes += L["w_ro"].numel() * 2
            if ls.mixer.branch_norm:
                L["left_out"], L["right_out"] = vec(p + "mix.left.out"), vec(p + "mix.right.out")
                if L["left_out"].numel() != W or L["right_out"].numel() != W:
                    raise ValueError(f"layer {i}: branch norm weights do not fit the width")
        self.max_proj = max(self.max_proj, L["w_in"].shape[0])
        f = ls.ff
        if f is not None:
            L["norm2"] = vec(p + "norm2")
            if L["norm2"].numel() != W:
                raise ValueError(f"layer {i}: norm weight does not fit the width")
        if isinstance(f, MoeFfSpec):
            self._load_moe(L, i, f, lin, vec, get)
        elif f is not None:
            if f.act != "polynorm":
                raise ValueError(f"layer {i}: dense feed-forward activation {f.act} is not wired into the out_norm layout")
            L["w_up"], L["w_down"], L["act_coef"] = lin(p + "mlp.up"), lin(p + "mlp.down"), vec(p + "mlp.act")
            if tuple(L["w_up"].shape) != (f.ff, W) or tuple(L["w_down"].shape) != (W, f.ff) or L["act_coef"].numel() != 4:
                raise ValueError(f"layer {i}: feed-forward tensor shapes do not fit the configuration")
            self.weight_bytes += (L["w_up"].numel() + L["w_down"].numel()) * 2
            self.max_ff_inner, self.max_ff_proj = max(self.max_ff_inner, f.ff), max(self.max_ff_proj, f.ff)
        return L

    def _load_moe(self, L, i: int, f: "MoeFfSpec", lin, vec, get) -> None:
        """tensors of a mixture-of-experts feed-forward: router (rows of a shared expert's token gate stacked behind it) or table, stacked expert
        weights (gated kinds with alternating gate / up rows), the shared expert"""
        cfg, W, p = self.cfg, self.cfg.width, f"l{i}."
        if f.act not in seqops.ACT_KINDS or not 1 <= f.top <= f.experts + f.identity:
            raise ValueError(f"layer {i}: expert activation {f.act} / top {f.top} is not supported")
        gated = seqops.ACT_KINDS[f.act] in seqops.ACT_GATED

        def gate_up(pre, ff):      # rows alternate (gate j, up j): the pair meets in one warp / neighbouring lanes
            gu = lin(pre + "gate", pre + "up")
            if tuple(gu.shape) != (2 * ff, W):
                raise ValueError(f"layer {i}: {pre}gate / up shapes do not fit the configuration")
            return gu.view(2, ff, W).transpose(0, 1).reshape(2 * ff, W).contiguous()

        if f.router == "table":
            t = get(p + "mlp.table")
            if t.dtype not in (torch.int32, torch.int64) or tuple(t.shape) != (cfg.vocab, f.top):
                raise ValueError(f"layer {i}: the expert table is an integer tensor [vocab, top]")
            if int(t.min()) < 0 or int(t.max()) >= f.experts:
                raise ValueError(f"layer {i}: the expert table names an expert outside 0..{f.experts - 1}")
            L["table"] = t.to(torch.int32).contiguous().to(self.dev)
        elif f.router in ("sigmoid", "softmax"):
            if f.router == "sigmoid" and (f.identity or f.correction):
                raise ValueError(f"layer {i}: identity experts and a correction go with the soft-max router")
            router = [p + "mlp.router"] + ([p + "mlp.shared.sg"] if f.shared_ff and f.shared_gate else [])
            L["w_router"] = lin(*router)
            if tuple(L["w_router"].shape) != (len(router) - 1 + f.experts + f.identity, W):
                raise ValueError(f"layer {i}: router shape does not fit the configuration")
            self.weight_bytes += L["w_router"].numel() * 2
            L["correction"] = vec(p + "mlp.correction") if f.correction else None
            if L["correction"] is not None and L["correction"].numel() != f.experts + f.identity:
                raise ValueError(f"layer {i}: one correction per router output expected")
        else:
            raise ValueError(f"layer {i}: unknown router kind {f.router}")
        if gated:
            L["w_eup"] = torch.stack([gate_up(p + f"mlp.e{e}.", f.ff) for e in range(f.experts)]).contiguous()
        else:
            L["w_eup"] = torch.stack([lin(p + f"mlp.e{e}.up") for e in range(f.experts)]).contiguous()
        L["w_edown"] = torch.stack([lin(p + f"mlp.e{e}.down") for e in range(f.experts)]).contiguous()
        if tuple(L["w_eup"].shape[1:]) != ((2 if gated else 1) * f.ff, W) or tuple(L["w_edown"].shape[1:]) != (W, f.ff):
            raise ValueError(f"layer {i}: expert tensor shapes do not fit the configuration")
        self.weight_bytes += (L["w_eup"].numel() + L["w_edown"].numel()) * 2
        if f.shared_ff:
            L["w_sup"] = gate_up(p + "mlp.shared.", f.shared_ff) if gated else lin(p + "mlp.shared.up")
            L["w_sdown"] = lin(p + "mlp.shared.down")
            if L["w_sup"].shape[1] != W or tuple(L["w_sdown"].shape) != (W, f.shared_ff):
                raise ValueError(f"layer {i}: shared expert tensor shapes do not fit the configuration")
            self.weight_bytes += (L["w_sup"].numel() + L["w_sdown"].numel()) * 2
            self.max_ff_inner = max(self.max_ff_inner, f.shared_ff)
            self.max_ff_proj = max(self.max_ff_proj, 2 * f.shared_ff)
        md = self.moe_dims or (1, 1, 1)
        self.moe_dims = (max(md[0], f.experts + f.identity + 1), max(md[1], f.top), max(md[2], f.ff))

    def _post_sizes(self, L, ls: "LayerSpec") -> None:
        """largest intermediates over the layers (workspace sizes)"""
        m, f = ls.mixer, ls.ff
        self.max_proj = max(self.max_proj, L["w_in"].shape[0])
        if ls.kind == "retention":
            self.max_inner = max(self.max_inner, m.heads * m.vdim)
        else:
            self.max_inner = max(self.max_inner, m.heads * m.vdim, m.heads * m.kv_rank, m.q_rank)
            self.max_q = max(self.max_q, m.heads * (m.dim + m.rot_dim), m.vdim)
            self.max_qp = max(self.max_qp, m.heads * (m.kv_rank + m.rot_dim))
            self.max_qn = max(self.max_qn, m.heads * m.dim)
            self.max_ctx_r, self.max_ctx_kv = max(self.max_ctx_r, m.kv_rank), max(self.max_ctx_kv, m.heads * (m.dim + m.vdim))
        if isinstance(f, MoeFfSpec):
            md = self.moe_dims or (1, 1, 1)
            self.moe_dims = (max(md[0], f.experts + 1), max(md[1], f.top), max(md[2], f.ff))
            if f.shared_ff:
                self.max_ff_inner = max(self.max_ff_inner, f.shared_ff)
                self.max_ff_proj = max(self.max_ff_proj, 2 * f.shared_ff)
        elif f is not None:
            self.max_ff_inner = max(self.max_ff_inner, f.ff)
            self.max_ff_proj = max(self.max_ff_proj, 2 * f.ff)

    # ---- cache and state -------------------------------------------------------------------------------------------------------
    def allocate(self, num_blocks: int, block_size: int, max_seqs: int, max_seq_tokens: int) -> None:
        """KV pools for `num_blocks` pages, state for `max_seqs` slots; block tables hold up to max_seq_tokens positions"""
        dev, cfg = self.dev, self.cfg
        f32 = dict(dtype=torch.float32, device=dev)
        self.block_size, self.max_seqs = block_size, max_seqs
        self.max_blocks = max(1, -(-max_seq_tokens // block_size))
        hist = cfg.canon_taps - 1
        for L in self.layers:
            ls = L["spec"]
            m = ls.mixer
            if cfg.layout == "streams":
                L["canon1_state"] = torch.zeros((max_seqs, max(hist, 1), cfg.width), **f32)
                if ls.ff is not None:
                    L["canon2_state"] = torch.zeros((max_seqs, max(hist, 1), cfg.width), **f32)
            if cfg.layout == "post":
                L["shift_state"] = torch.zeros((max_seqs, cfg.width), **f32)      # the mixer input of the sequence's last token
            if cfg.layout == "out_norm":
                att = m if ls.kind == "attention" else m.left
                maps = 2 if att.diff is not None else 1
                if att.kv_from is None:      # a layer that reads another layer's keys and values has no pool (bound below, when all pools exist)
                    L["kpool"] = torch.zeros((max(1, num_blocks), block_size, att.kv_heads * maps, att.dim), **f32)
                    L["vpool"] = torch.zeros((max(1, num_blocks), block_size, att.kv_heads, att.vdim), **f32)
                right = None if ls.kind == "attention" else m.right
                if isinstance(right, MinGruSpec):
                    L["rec_state"] = torch.zeros((max_seqs, right.width), **f32)
                elif isinstance(right, RgLruSpec):
                    L["rec_state"] = torch.zeros((max_seqs, right.width), **f32)
                    L["conv_state"] = torch.zeros((max_seqs, max(right.conv - 1, 1), right.width), **f32)
                continue
            if ls.kind == "retention":
                L["ret_state"] = torch.zeros((max_seqs, m.heads, m.dim, m.vdim), **f32)
            elif ls.kind == "latent_attention":       # one row [latent | rotated key part] per position; keys and values of all heads come out of it
                L["kpool"] = torch.zeros((max(1, num_blocks), block_size, m.kv_rank + m.rot_dim), **f32)
                L["desc_x"] = seqops.expanded_attn_desc(m.heads, m.dim, m.rot_dim, m.vdim, m.scale, L["kpool"].view(-1, m.kv_rank + m.rot_dim)[:, m.kv_rank:],
                                                        gated=m.gated, sink=L["sink"])
            elif ls.kind == "attention":
                L["kpool"] = torch.zeros((max(1, num_blocks), block_size, m.kv_heads, m.dim), **f32)
                L["vpool"] = torch.zeros((max(1, num_blocks), block_size, m.kv_heads, m.vdim), **f32)
                if m.pool > 0:      # mean key / value of every block of `pool` positions, kept in the page of the block's first position
                    per_page = -(-block_size // m.pool)
                    L["kpooled"] = torch.zeros((max(1, num_blocks), per_page, m.kv_heads, m.dim), **f32)
                    L["vpooled"] = torch.zeros((max(1, num_blocks), per_page, m.kv_heads, m.vdim), **f32)
            else:
                L["conv_state"] = torch.zeros((max_seqs, max(m.conv - 1, 1), m.heads * m.vdim + 2 * m.groups * m.state), **f32)
                L["ssm_state"] = torch.zeros((max_seqs, m.heads, m.state, m.vdim), **f32)
        if cfg.layout == "out_norm":
            for L in self.layers:
                att = L["spec"].mixer if L["spec"].kind == "attention" else L["spec"].mixer.left
                L["kv_src"] = self.layers[att.kv_from] if att.kv_from is not None else L
        self._ws.clear()
        self._graphs.clear()

    def scratch_floats(self, cap: int) -> int:
        """floats of the largest work area any layer wants for a step of up to `cap` tokens"""
        need = 0
        seen = set()
        for L in self.layers:
            m = L["spec"].mixer
            if self.cfg.layout == "out_norm":
                att = m if L["spec"].kind == "attention" else m.left
                maps = 2 if att.diff is not None else 1
                ctx = keys = self.max_blocks * self.block_size
                if att.window > 0:
                    keys = min(ctx, att.window + att.keep_first)
                key = (att.heads * maps, att.kv_heads * maps, att.vdim, keys)
                if key not in seen:
                    seen.add(key)
                    need = max([need] + [seqops.attn_scratch_floats(T, 1, key[0], key[1], att.vdim, keys) for T in range(1, cap + 1)])
                continue
            if L["spec"].kind == "ssm":
                need = max(need, seqops.ssm_scratch_floats(cap, self.max_seqs, m.heads, m.vdim, m.state))
            elif L["spec"].kind == "retention":
                need = max(need, seqops.retention_scratch_floats(cap, self.max_seqs, m.heads, m.dim, m.vdim))
            elif L["spec"].kind == "latent_attention":
                key = ("latent", m.heads, m.kv_rank)
                if key not in seen:
                    seen.add(key)
                    ctx = self.max_blocks * self.block_size
                    need = max([need] + [max(seqops.attn_scratch_floats(T, 1, m.heads, 1, m.kv_rank, ctx), seqops.attn_scratch_floats(T, 1, m.heads, m.heads, m.vdim, ctx))
                                         for T in range(1, cap + 1)])
            else:
                ctx = keys = self.max_blocks * self.block_size
                keys = min(keys, m.chunk) if m.chunk > 0 else keys
                keys = min(keys, m.window) if m.window > 0 else keys
                keys += ctx // m.pool if m.pool > 0 else 0
                key = (m.heads, m.kv_heads, m.vdim, keys)
                if key not in seen:     # the split count falls as the step grows: the largest need is at some T <= cap
                    seen.add(key)
                    need = max([need] + [seqops.attn_scratch_floats(T, 1, m.heads, m.kv_heads, m.vdim, keys) for T in range(1, cap + 1)])
        return need

    def cache_bytes(self) -> int:
        keys = ("canon1_state", "canon2_state", "kpool", "vpool", "kpooled", "vpooled", "conv_state", "ssm_state", "shift_state", "ret_state", "rec_state")
        return sum(L[k].numel() * 4 for L in self.layers for k in keys if k in L)

    def _ctx_buffers(self, rows: int):
        """gathered latents (activation type) and the per-head keys | values projected out of them (f32) for `rows` context positions;
        grown on demand, shared by all latent-attention layers"""
        cap = 256
        while cap < rows:
            cap *= 2
        if self._ctx_cap < cap:
            self._ctx = (torch.empty((cap, self.max_ctx_r), dtype=self.act_dtype, device=self.dev), torch.empty((cap, self.max_ctx_kv), dtype=torch.float32, device=self.dev))
            self._ctx_cap = cap
        return self._ctx

    def _workspace(self, T: int) -> _Workspace:
        cap = 8
        while cap < T:
            cap *= 2
        ws = self._ws.get(cap)
        if ws is None:
            ws = self._ws[cap] = _Workspace(self, cap)
        return ws

    # ---- the step ----------------------------------------------------------------------------------------------------------------
    def _upload(self, ws: _Workspace, sa: StepArrays) -> None:
        if sa.B > self.max_seqs or sa.block_table.shape[1] > self.max_blocks:
            raise ValueError("step exceeds the engine's request or block-table capacity")
        h = ws.meta_host
        if ws.copied is not None:
            ws.copied.synchronize()    # the previous step's copy out of the pinned buffer must be over before it is rewritten
        hn = h.numpy()
        prev = sa.ent_prev if sa.ent_prev is not None else np.zeros(sa.B, dtype=np.int32)
        for k, arr in (("ids", sa.tok_ids), ("ent", sa.tok_ent), ("pos", sa.tok_pos), ("want", sa.want_rows), ("start", sa.ent_start), ("slot", sa.ent_slot),
                       ("pos0", sa.ent_pos0), ("prev", prev)):
            o, _ = ws.off[k]
            hn[o:o + arr.shape[0]] = arr
        o, _ = ws.off["bt"]
        bt = np.zeros((sa.B, self.max_blocks), dtype=np.int32)
        bt[:, :sa.block_table.shape[1]] = sa.block_table
        hn[o:o + bt.size] = bt.reshape(-1)
        ws.meta.copy_(h, non_blocking=True)
        if self.dev.type == "cuda":
            ws.copied = torch.cuda.Event()
            ws.copied.record(torch.cuda.current_stream(self.dev))

    def _desc(self, ws: _Workspace, T: int, B: int) -> seqops.StepDesc:
        ptr = lambda k: ws.view(k).data_ptr()
        return seqops.StepDesc(ptr("ent"), ptr("pos"), ptr("start"), ptr("slot"), ptr("pos0"), ptr("bt"), T, B, self.max_blocks, self.block_size)

    def forward(self, sa: StepArrays, sample: bool = False, debug_layers: Optional[list] = None) -> torch.Tensor:
        """runs one step; returns f32 logits [R, vocab] of the wanted rows (a view of a buffer the next step overwrites);
        sample: also leaves the greedy token of every wanted row in `self.last_ids` (int32 [R], device)"""
        if not self.block_size:
            raise RuntimeError("allocate() the cache first")
        T, B, R = sa.T, sa.B, int(sa.want_rows.shape[0])
        self._ctx_rows = int(sa.ent_pos0.sum()) + T if (T > B and self.max_ctx_r) else 0
        ws = self._workspace(T)
        self._upload(ws, sa)
        graphable = self.use_graphs and debug_layers is None and sa.decode_only and R == T and self.dev.type == "cuda" \
            and bool((sa.want_rows == np.arange(T)).all())
        if graphable:
            key = (T, bool(sample))
            g = self._graphs.get(key)
            if g is None:
                self._run(ws, T, B, R, sample, None)        # warm-up outside capture (module loading, attribute calls)
                torch.cuda.synchronize(self.dev)
                # the warm-up run advanced the carried state: capture must not run it twice -> capture on a side stream, then the
                # captured launches are NOT executed; state was advanced exactly once by the warm-up.
                g = torch.cuda.CUDAGraph()
                s = torch.cuda.Stream(self.dev)
                s.wait_stream(torch.cuda.current_stream(self.dev))
                with torch.cuda.stream(s):
                    with torch.cuda.graph(g, stream=s):
                        self._run(ws, T, B, R, sample, None)
                torch.cuda.current_stream(self.dev).wait_stream(s)
                self._graphs[key] = g
            else:
                g.replay()
        else:
            self._run(ws, T, B, R, sample, debug_layers)
        self.last_ids = ws.next_ids[:R]
        return ws.logits[:R]

    def _run(self, ws: _Workspace, T: int, B: int, R: int, sample: bool, debug_layers: Optional[list]) -> None:
        if self.cfg.layout == "depth":
            self._run_depth(ws, T, B, R, sample, debug_layers)
        elif self.cfg.layout == "post":
            self._run_post(ws, T, B, R, debug_layers)
        elif self.cfg.layout == "out_norm":
            self._run_out(ws, T, B, R, debug_layers)
        else:
            self._run_streams(ws, T, B, R, sample, debug_layers)
        if R:
            seqops.linear(ws.fin[:R], self.head, ws.logits[:R])
            if self.cfg.logit_softcap > 0:
                seqops.softcap(ws.logits[:R], self.cfg.logit_softcap)
            if sample:
                seqops.argmax(ws.logits[:R], ws.next_ids[:R])

    def _run_depth(self, ws: _Workspace, T: int, B: int, R: int, sample: bool, debug_layers: Optional[list]) -> None:
        """parallel layers over one depth-averaged residual stream.  Between two layers one kernel adds the two branches to the layer's
        input, stores the result for the averages to come, forms the next layer's input and applies both of its layer norms."""
        cfg, ops = self.cfg, seqops
        st = self._desc(ws, T, B)
        hist, xbuf = ws.hist, ws.xbuf[:T]
        a1, a2, y1, y2 = ws.a[:T], ws.a2[:T], ws.y[:T], ws.y2[:T]
        x0 = hist[0, :T]
        ops.embed_streams(self.embed, ws.view("ids"), cfg.embed_scale, x0.view(T, 1, cfg.width))
        n = len(self.layers)
        if n:
            L0 = self.layers[0]
            ops.depth_norm(x0, a1, L0["norm1"], cfg.eps, out2=a2 if L0["spec"].ff is not None else None, w2=L0.get("norm2"))
        x_cur = x0
        # the two branches of a layer read the same input and do not depend on one another: the feed-forward runs on a second stream
        # beside the mixer, a shared expert on a third beside the routed ones (inside a captured decode step they become parallel branches
        # of the graph).  Not while operators are timed alone.
        two_streams = self.overlap_branches and self.dev.type == "cuda" and seqops.timeline is None
        if two_streams and self._side is None:
            self._side, self._side2 = torch.cuda.Stream(self.dev), torch.cuda.Stream(self.dev)
        for i, L in enumerate(self.layers):
            ls: LayerSpec = L["spec"]
            if ls.kind != "attention":
                raise ValueError("the depth-averaged layout is wired for attention mixers")
            has_ff = ls.ff is not None

            def feed_forward(shared_done=None):
                if isinstance(ls.ff, MoeFfSpec):
                    self._moe_ff(L, ls.ff, ws, T, a2, y2, shared_done)
                else:
                    self._dense_ff(L, ls.ff, ws, T, a2, y2, inner=ws.ff_inner, proj=ws.ff_proj)

            if has_ff and two_streams:
                main = torch.cuda.current_stream(self.dev)
                fork, join = torch.cuda.Event(), torch.cuda.Event()
                fork.record(main)
                shared_done = None
                if isinstance(ls.ff, MoeFfSpec) and ls.ff.shared_ff:      # the shared expert does not wait for the router either: a third stream
                    shared_done = torch.cuda.Event()
                    self._side2.wait_event(fork)
                    with torch.cuda.stream(self._side2):
                        self._shared_expert(L, ls.ff, ws, T, a2)
                        shared_done.record(self._side2)
                self._side.wait_event(fork)
                with torch.cuda.stream(self._side):
                    feed_forward(shared_done)
                    join.record(self._side)
                self._attention(L, ls.mixer, ws, st, T, a1, y1)
                main.wait_event(join)
            else:
                self._attention(L, ls.mixer, ws, st, T, a1, y1)
                if has_ff:
                    feed_forward()
            upd = dict(y1=y1, y2=y2 if has_ff else None, hist=hist, n_prev=i + 1, dwa=L["dwa"], x_out=xbuf)
            if i + 1 < n:
                N = self.layers[i + 1]
                two = N["spec"].ff is not None
                ops.depth_norm(x_cur, a1, N["norm1"], cfg.eps, out2=a2 if two else None, w2=N.get("norm2") if two else None, hist_out=hist[i + 1, :T], **upd)
            elif debug_layers is not None:
                ops.depth_norm(x_cur, None, None, cfg.eps, **upd)
                if R:
                    ops.depth_norm(xbuf, ws.fin[:R], self.final_norm, cfg.eps, rows=ws.view("want")[:R])
            elif R:
                ops.depth_norm(x_cur, ws.fin[:R], self.final_norm, cfg.eps, rows=ws.view("want")[:R], **upd)
            x_cur = xbuf
            if debug_layers is not None:
                debug_layers.append(xbuf.cpu())
        if not n and R:
            ops.depth_norm(x0, ws.fin[:R], self.final_norm, cfg.eps, rows=ws.view("want")[:R])

    def _run_post(self, ws: _Workspace, T: int, B: int, R: int, debug_layers: Optional[list]) -> None:
        """sublayers in sequence over one residual x (f32): mixer(shifted x) and feed-forward(x), each times sigmoid(rg x + b), each followed by
        the layer norm of alpha x + gated result.  Between sublayers ONE kernel: gate, sum, norm, the next sublayer's input in the activation type,
        the shift state of the mixer it closes and - in steps of single tokens - the token shift of the next mixer."""
        cfg, ops = self.cfg, seqops
        st = self._desc(ws, T, B)
        x, a, ash, y, zg = ws.h[:T], ws.a[:T], ws.a2[:T], ws.y[:T], ws.zg[:T]
        ops.embed_streams(self.embed, ws.view("ids"), cfg.embed_scale, x.view(T, 1, cfg.width))
        n = len(self.layers)
        single = T == B
        # What does not lie on a sublayer's critical path runs beside it on other streams (inside a captured decode step: parallel branches of
        # the graph): the residual gate's projection beside the mixer / the experts, the shared expert on a third stream, and - because a
        # table-routed choice depends on the token ids alone - the choice and the sort of EVERY layer at the start of the step.
        par = self.overlap_branches and self.dev.type == "cuda" and seqops.timeline is None
        if par and self._side is None:
            self._side, self._side2 = torch.cuda.Stream(self.dev), torch.cuda.Stream(self.dev)
        main = torch.cuda.current_stream(self.dev) if par else None

        def beside(stream, fn):
            """fn on `stream` after what the main stream has queued so far; returns the event to wait for (None: it ran in line)"""
            if not par:
                fn()
                return None
            fork, done = torch.cuda.Event(), torch.cuda.Event()
            fork.record(main)
            stream.wait_event(fork)
            with torch.cuda.stream(stream):
                fn()
                done.record(stream)
            return done

        def wait(ev):
            if ev is not None:
                main.wait_event(ev)

        tabled = [i for i, L in enumerate(self.layers) if isinstance(L["spec"].ff, MoeFfSpec) and L["spec"].ff.router == "table"]
        routed = beside(self._side2 if par else None, lambda: [self._table_route(self.layers[i], ws, i, T) for i in tabled]) if tabled else None
        if n:
            ops.token_shift(x, self.layers[0]["shift"], self.layers[0]["shift_state"], st, a, ash)
        for i, L in enumerate(self.layers):
            ls: LayerSpec = L["spec"]
            gate_done = beside(self._side, lambda: ops.linear(a, L["rg1"], zg))
            if ls.kind == "retention":
                self._retention(L, ls.mixer, ws, st, T, ash, y)
            else:
                self._latent_attention(L, ls.mixer, ws, st, T, ash, y)
            close = dict(y=y, zg=zg, alpha=cfg.post_alpha, x_out=x, a_out=a, step=st)
            q = 1
            if ls.ff is not None:
                wait(gate_done)
                ops.post_norm(x, L["norm1"], L["norm1_b"], cfg.eps, gate_b=L["rg1_b"], state_out=L["shift_state"], **close)
                gate_done = beside(self._side, lambda: ops.linear(a, L["rg2"], zg))
                if isinstance(ls.ff, MoeFfSpec):
                    shared_done = None
                    if par and ls.ff.shared_ff:
                        shared_done = beside(self._side2, lambda: self._shared_expert(L, ls.ff, ws, T, a))
                    if i in tabled:
                        wait(routed)
                        routed = None
                    self._moe_ff(L, ls.ff, ws, T, a, y, shared_done, route=ws.route.get(i))
                else:
                    self._dense_ff(L, ls.ff, ws, T, a, y, inner=ws.ff_inner, proj=ws.ff_proj)
                q = 2
            else:
                close["state_out"] = L["shift_state"]
            nxt = self.layers[i + 1] if i + 1 < n else None
            if nxt is not None and single:
                close.update(next_mu=nxt["shift"], next_state=nxt["shift_state"], a_shift_out=ash)
            wait(gate_done)
            ops.post_norm(x, L[f"norm{q}"], L[f"norm{q}_b"], cfg.eps, gate_b=L[f"rg{q}_b"], **close)
            if nxt is not None and not single:
                ops.token_shift(x, nxt["shift"], nxt["shift_state"], st, None, ash)
            if debug_layers is not None:
                debug_layers.append(x.cpu())
        wait(routed)
        if R:
            ops.post_norm(x, self.final_norm, self.final_bias, cfg.eps, rows=ws.view("want")[:R], a_out=ws.fin[:R])

    def _run_out(self, ws: _Workspace, T: int, B: int, R: int, debug_layers: Optional[list]) -> None:
        """sublayers in sequence over one residual x (f32) that they read as it is; between sublayers ONE kernel sums the mixer's branches (with
        their scales, output bias and branch norms), applies the norm on the sublayer's output, adds the residual and writes the next sublayer's
        input in the activation type; after the last sublayer the same kernel applies the final norm to the wanted rows."""
        cfg, ops = self.cfg, seqops
        st = self._desc(ws, T, B)
        x, a, y, y2 = ws.h[:T], ws.a[:T], ws.y[:T], ws.y2[:T]
        bg = cfg.bigram or (0, 0, 0)
        ops.embed_bigram(self.embed, self.bigram, ws.view("ids"), ws.view("prev"), st, cfg.embed_scale, int(bg[0]), int(bg[1]), int(bg[2]), x, a)
        n = len(self.layers)
        want = ws.view("want")[:R]
        # The two branches of a mixer read the same projection and do not depend on one another: the recurrent one runs on a second stream
        # beside the attention, a shared expert on a third beside the routed ones (inside a captured decode step they become parallel
        # branches of the graph).  Not while operators are timed alone.
        par = self.overlap_branches and self.dev.type == "cuda" and seqops.timeline is None
        if par and self._side is None:
            self._side, self._side2 = torch.cuda.Stream(self.dev), torch.cuda.Stream(self.dev)
        main = torch.cuda.current_stream(self.dev) if par else None

        def beside(stream, fn):
            """fn on `stream` after what the main stream has queued so far; returns the event to wait for (None: it ran in line)"""
            if not par:
                fn()
                return None
            fork, done = torch.cuda.Event(), torch.cuda.Event()
            fork.record(main)
            stream.wait_event(fork)
            with torch.cuda.stream(stream):
                fn()
                done.record(stream)
            return done

        def close(L, q, last, **branches):
            """x <- x + norm_q(branches); the last sublayer of the model leaves the final norm of the wanted rows instead of the next input"""
            if last and debug_layers is None:
                if R:
                    ops.branch_norm(x, w=L[f"norm{q}"], eps=cfg.eps, rows=want, a_out=ws.fin[:R], fin_w=self.final_norm, **branches)
                return
            ops.branch_norm(x, w=L[f"norm{q}"], eps=cfg.eps, x_out=x, a_out=a, **branches)

        for i, L in enumerate(self.layers):
            ls: LayerSpec = L["spec"]
            proj = ws.proj[:T, :L["w_in"].shape[0]]
            ops.linear(a, L["w_in"], proj)
            has_ff = ls.ff is not None
            last = i + 1 == n
            if ls.kind == "attention":
                self._attention_out(L, ls.mixer, ws, st, T, proj, y)
                close(L, 1, last and not has_ff, y1=y, bias1=L["o_bias"])
            else:
                tb: TwoBranchSpec = ls.mixer
                right_done = beside(self._side, lambda: self._recurrent_branch(L, tb.right, ws, st, T, proj, y2))
                self._attention_out(L, tb.left, ws, st, T, proj, y)
                if right_done is not None:
                    main.wait_event(right_done)
                close(L, 1, last and not has_ff, y1=y, bias1=L["o_bias"], w_b1=L.get("left_out"), s1=tb.left_scale, y2=y2, w_b2=L.get("right_out"), s2=tb.right_scale)
            if has_ff:
                if isinstance(ls.ff, MoeFfSpec):
                    shared_done = beside(self._side2, lambda: self._shared_expert(L, ls.ff, ws, T, a)) if par and ls.ff.shared_ff else None
                    self._moe_ff(L, ls.ff, ws, T, a, y, shared_done, x_id=x)
                else:
                    z = ws.ff_proj.view(-1)[:T * ls.ff.ff].view(T, ls.ff.ff)
                    ops.linear(a, L["w_up"], z)
                    mid = ws.ff_inner.view(-1)[:T * ls.ff.ff].view(T, ls.ff.ff)
                    ops.polynorm(z, L["act_coef"], cfg.eps, mid)
                    ops.linear(mid, L["w_down"], y)
                close(L, 2, last, y1=y)
            if debug_layers is not None:
                debug_layers.append(x.cpu())
        if R and (not n or debug_layers is not None):
            ops.group_rmsnorm(x if R == T and debug_layers is None else x.index_select(0, want.long()), self.final_norm, 1, cfg.eps, ws.fin[:R])

    def _attention_out(self, L, m: AttentionSpec, ws: _Workspace, st, T: int, proj: torch.Tensor, y: torch.Tensor) -> None:
        """attention of the out_norm layout over the layer's own pool or the pool of the layer whose keys and values it shares"""
        src = L["kv_src"]
        seqops.attn_prep_ex(proj, st, L["desc"], L.get("kpool"), L.get("vpool"))
        H, V = m.heads, m.vdim
        o = ws.inner_a.view(-1)[:T * H * V].view(T, H * V)
        if m.diff is not None:      # two maps per head as 2 H plain heads, f32; then o = unit_rms(a1 - lambda a2) * (1 - diff)
            a12 = ws.inner_f.view(-1)[:T * 2 * H * V].view(T, 2 * H * V)
            seqops.attn_ex(proj, st, L["desc"], src["kpool"], src["vpool"], a12, ws.scratch)
            seqops.diff_combine(a12, H, m.kv_heads, V, L["lambda"], 1.0 - m.diff, self.cfg.eps, o)
        else:
            seqops.attn_ex(proj, st, L["desc"], src["kpool"], src["vpool"], o, ws.scratch)
        seqops.linear(o, L["w_o"], y)

    def _recurrent_branch(self, L, r, ws: _Workspace, st, T: int, proj: torch.Tensor, y: torch.Tensor) -> None:
        rc, C = L["rcols"], r.width
        out = ws.inner_b.view(-1)[:T * C].view(T, C)
        if isinstance(r, MinGruSpec):
            seqops.min_gru(proj, rc["z"], rc["x"], rc["g"], L["in_bias"], L["rec_state"], st, C, out)
        else:
            u = ws.xbc.view(-1)[:T * C].view(T, C)
            ua = ws.conv_a.view(-1)[:T * C].view(T, C)
            seqops.causal_conv_ex(proj[:, rc["x"]:rc["x"] + C], L["x_bias"], L["conv_w"], L["conv_b"], L["conv_state"], st, 0, u, ua)
            gates = ws.gates.view(-1)[:T * 2 * C].view(T, 2 * C)
            bw = C // r.blocks
            seqops.head_linear(ua, L["w_gates"], gates, 2 * bw)
            seqops.rg_lru(u, gates, L["gate_bias"], L["sp_lam"], r.decay, proj, rc["y"], L["in_bias"], L["rec_state"], st, r.blocks, out)
        seqops.linear(out, L["w_ro"], y)

    def _retention(self, L, m: RetentionSpec, ws: _Workspace, st, T: int, a: torch.Tensor, y: torch.Tensor) -> None:
        proj = ws.proj[:T, :L["w_in"].shape[0]]
        seqops.linear(a, L["w_in"], proj)
        o = ws.inner_a.view(-1)[:T * m.heads * m.vdim].view(T, m.heads * m.vdim)
        seqops.retention(proj, st, L["desc"], L["ret_state"], o, ws.scratch)
        seqops.linear(o, L["w_o"], y)

    def _latent_attention(self, L, m: LatentAttentionSpec, ws: _Workspace, st, T: int, a: torch.Tensor, y: torch.Tensor) -> None:
        """Two forms with the same result.  Single-token steps stay in the latent space (the cache is read as it is: H query heads of size
        kv_rank + rot_dim over one key head).  Steps with prompt portions gather the latents of the entries' contexts, project per-head keys and
        values out of them once, and attend with heads of size dim + rot_dim: far fewer operations per (query, key) pair."""
        H, Dn, Rd, V, R, Rq = m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank
        eps = self.cfg.eps
        proj = ws.proj[:T, :L["w_in"].shape[0]]
        seqops.linear(a, L["w_in"], proj)                                   # c_q | c, k_rot | gate logits
        cq = ws.inner_a.view(-1)[:T * Rq].view(T, Rq)
        seqops.group_rmsnorm(proj[:, :Rq], L["dq_norm"], 1, eps, cq)
        q = ws.q.view(-1)[:T * H * (Dn + Rd)].view(T, H * (Dn + Rd))
        seqops.linear(cq, L["w_uq"], q)
        gate = proj[:, Rq + R + Rd:] if m.gated else None
        if self._ctx_rows > 0:
            ctx = self._ctx_rows
            seqops.latent_prep(proj, Rq, -1, q, st, H, Dn, Rd, R, L["kv_norm"], eps, L["rot_freq"], L["rot_scale"], L["kpool"], None, None)
            cx, kvx = self._ctx_buffers(ctx)
            cx = cx.view(-1)[:ctx * R].view(ctx, R)
            kvx = kvx.view(-1)[:ctx * H * (Dn + V)].view(ctx, H * (Dn + V))
            seqops.latent_gather(L["kpool"], st, R, ctx, cx)
            seqops.linear(cx, L["w_ukv"], kvx)
            up = ws.oup.view(-1)[:T * H * V].view(T, H * V)
            seqops.attn_ex(q, st, L["desc_x"], kvx, kvx[:, H * Dn:], up, ws.scratch, gate=gate)
            seqops.linear(up, L["w_o"], y)
            return
        Qp = ws.Qp.view(-1)[:T * H * (R + Rd)].view(T, H * (R + Rd))
        qn = ws.qn.view(-1)[:T * H * Dn].view(T, H * Dn)
        seqops.latent_prep(proj, Rq, -1, q, st, H, Dn, Rd, R, L["kv_norm"], eps, L["rot_freq"], L["rot_scale"], L["kpool"], Qp, qn)
        # the unrotated query parts enter the latent space head by head: Qp[t][h][:R] = W_uk[h]^T q_nope[t][h]
        seqops.head_linear(qn, L["w_ukT"], Qp, R + Rd)
        o = ws.inner_a.view(-1)[:T * H * R].view(T, H * R)
        seqops.attn_ex(Qp, st, L["desc"], L["kpool"], None, o, ws.scratch, gate=gate)
        up = ws.oup.view(-1)[:T * H * V].view(T, H * V)
        seqops.head_linear(o, L["w_uv"], up, V, seqops.ACT_IDENT)      # values leave the latent space after the weighted sum
        seqops.linear(up, L["w_o"], y)

    def _run_streams(self, ws: _Workspace, T: int, B: int, R: int, sample: bool, debug_layers: Optional[list]) -> None:
        cfg = self.cfg
        ops = seqops
        st = self._desc(ws, T, B)
        X, h, a, y = ws.X[:T], ws.h[:T], ws.a[:T], ws.y[:T]
        ops.embed_streams(self.embed, ws.view("ids"), cfg.embed_scale, X)
        y_prev = post_prev = None
        for L in self.layers:
            ls: LayerSpec = L["spec"]
            for q in ((1, 2) if ls.ff is not None else (1,)):
                if T == B:      # one token per entry: the convolution's history is all in the carried state -> one kernel
                    ops.hc_norm_conv(X, y_prev, post_prev, L[f"hc{q}_in"], L[f"norm{q}"], cfg.norm_groups, cfg.eps, L[f"canon{q}"], L[f"canon{q}_state"], st, a)
                else:
                    ops.hc_norm(X, y_prev, post_prev, L[f"hc{q}_in"], L[f"norm{q}"], cfg.norm_groups, cfg.eps, h)
                    ops.causal_conv(h, L[f"canon{q}"], None, L[f"canon{q}_state"], st, ops.CONV_RESIDUAL, a)
                if q == 2:
                    self._dense_ff(L, ls.ff, ws, T, a, y)
                elif ls.kind == "attention":
                    self._attention(L, ls.mixer, ws, st, T, a, y)
                else:
                    self._ssm(L, ls.mixer, ws, st, T, a, y)
                y_prev, post_prev = y, L[f"hc{q}_post"]
            if debug_layers is not None:   # the streams' sum after this layer (the pending stream update applied on a copy)
                S = cfg.streams
                outv, mix = post_prev[:S], post_prev[S:].reshape(S, S)
                Xn = torch.einsum("st,nsw->ntw", mix, X) + outv[None, :, None] * y[:, None, :]
                debug_layers.append(Xn.sum(1).cpu())
        if R:
            ops.hc_norm(X, y_prev, post_prev, self.ones_in, self.final_norm, cfg.norm_groups, cfg.eps, ws.fin[:R], rows=ws.view("want")[:R])

    def _attention(self, L, m: AttentionSpec, ws: _Workspace, st, T: int, a: torch.Tensor, y: torch.Tensor) -> None:
        n_in = L["w_in"].shape[0]
        qkvg = ws.proj[:T, :n_in]
        seqops.linear(a, L["w_in"], qkvg)
        seqops.attn_prep_ex(qkvg, st, L["desc"], L["kpool"], L["vpool"], L.get("kpooled"), L.get("vpooled"))
        o = ws.inner_a.view(-1)[:T * m.heads * m.vdim].view(T, m.heads * m.vdim)
        seqops.attn_ex(qkvg, st, L["desc"], L["kpool"], L["vpool"], o, ws.scratch, L.get("kpooled"), L.get("vpooled"))
        seqops.linear(o, L["w_o"], y)

    def _ssm(self, L, m: SsmSpec, ws: _Workspace, st, T: int, a: torch.Tensor, y: torch.Tensor) -> None:
        inner, gn = m.heads * m.vdim, m.groups * m.state
        n_in = 2 * inner + 2 * gn + m.heads
        proj = ws.proj[:T, :n_in]
        seqops.linear(a, L["w_in"], proj)
        xbc = ws.xbc.view(-1)[:T * (inner + 2 * gn)].view(T, inner + 2 * gn)
        seqops.causal_conv(proj[:, inner:2 * inner + 2 * gn], L["conv_w"], L["conv_b"], L["conv_state"], st, seqops.CONV_SILU, xbc)
        yg = ws.inner_f.view(-1)[:T * inner].view(T, inner)
        seqops.ssm_scan(proj, 0, 2 * inner + 2 * gn, xbc, L["A_log"], L["D"], L["dt_bias"], L["ssm_state"], st, m.heads, m.vdim, m.state, m.groups, yg, ws.scratch)
        yn = ws.inner_a.view(-1)[:T * inner].view(T, inner)
        seqops.group_rmsnorm(yg, L["mnorm"], m.norm_groups, self.cfg.eps, yn)
        seqops.linear(yn, L["w_o"], y)

    def _dense_ff(self, L, f: DenseFfSpec, ws: _Workspace, T: int, a: torch.Tensor, y: torch.Tensor, inner: Optional[torch.Tensor] = None,
                  proj: Optional[torch.Tensor] = None) -> None:
        inner = ws.inner_a if inner is None else inner
        act = inner.view(-1)[:T * f.ff].view(T, f.ff)
        self._proj_act(ws.proj if proj is None else proj, T, a, L["w_gu"], seqops.ACT_KINDS[f.act], act, f.limit, f.alpha, f.up_shift)
        seqops.linear(act, L["w_down"], y)

    def _proj_act(self, proj: torch.Tensor, T: int, a: torch.Tensor, w: torch.Tensor, kind: int, out: torch.Tensor, limit: float = 0.0, alpha: float = 0.0,
                  shift: float = 0.0) -> None:
        """out = act(a . w^T): projection and activation in one kernel where a fused path takes the step, else product (in `proj`) + activation"""
        if T <= 8 or (T >= seqops.TC_MIN_ROWS and seqops.tc_usable(a, a.shape[1])):
            seqops.linear_act(a, w, kind, out, limit, alpha, shift)
        else:
            z = proj[:T, :w.shape[0]]
            seqops.linear(a, w, z)
            seqops.act(z, kind, out, limit, alpha, shift)

    def _table_route(self, L, ws: _Workspace, i: int, T: int) -> None:
        """choice (and, for many pairs, the sort by expert) of layer i's table-routed experts into the layer's own buffers: it needs the token ids only"""
        f, r = L["spec"].ff, ws.route[i]
        pairs = T * f.top
        rows_form = pairs <= self.MOE_ROW_PAIRS
        seqops.moe_table_route(L["table"], ws.view("ids"), T, f.experts, f.top, r["ids"], r["wts"], None if rows_form else r["cnt"])
        if not rows_form:
            seqops.moe_sort(r["ids"], pairs, f.experts, r["cnt"], r["off"], r["order"], r["slot"])

    MOE_ROW_PAIRS = 64      # up to this many (token, choice) pairs the experts' weights are streamed per pair; more: tiles over sorted pairs

    def _moe_ff(self, L, f: "MoeFfSpec", ws: _Workspace, T: int, a: torch.Tensor, y: torch.Tensor, shared_done=None, route=None, x_id=None) -> None:
        """shared_done: event after which the shared expert's output is in ws.moe_sh (it ran elsewhere); None: it runs here.
        route: the layer's own choice buffers, filled (and sorted) earlier in the step (table-routed layers); None: the choice is made here"""
        ops = seqops
        E, top = f.experts + f.identity, f.top      # E: router outputs (identity experts behind the real ones: they take part in the choice and the sort)
        gated_shared = bool(f.shared_ff and f.shared_gate)
        pairs = T * top
        rows_form = pairs <= self.MOE_ROW_PAIRS
        z = None
        ids, wts = (route["ids"], route["wts"]) if route is not None else (ws.moe_ids, ws.moe_wts)
        if route is not None:
            pass
        elif f.router == "table":         # no router: the token id names the experts
            ops.moe_table_route(L["table"], ws.view("ids"), T, E, top, ids, wts, None if rows_form else ws.moe_cnt)
        elif f.router == "softmax":
            z = ws.moe_z[:T, :L["w_router"].shape[0]]
            if T <= 8 and rows_form:        # few tokens: projection and choice in one kernel
                ops.moe_router_ex(a, L["w_router"], E, 1, 1, top, ops.ROUTE_SOFTMAX, L["correction"], z, ids, wts)
            else:
                ops.linear(a, L["w_router"], z)
                ops.moe_route_ex(z, E, 1, 1, top, ops.ROUTE_SOFTMAX, L["correction"], ids, wts, None if rows_form else ws.moe_cnt)
        else:
            z = ws.moe_z[:T, :L["w_router"].shape[0]]
            if T <= 8 and rows_form:        # few tokens: projection and choice in one kernel
                ops.moe_router(a, L["w_router"], E, f.groups, f.keep, top, z, ids, wts)
            else:
                ops.linear(a, L["w_router"], z)
                ops.moe_route(z, E, f.groups, f.keep, top, ids, wts, None if rows_form else ws.moe_cnt)
        kind = ops.ACT_KINDS[f.act]
        mid = ws.moe_act.view(-1)[:pairs * f.ff].view(pairs, f.ff)
        act_args = (f.limit, f.alpha, f.up_shift) if kind in ops.ACT_GATED else ()     # gated experts: activation of the (gate, up) pairs in the projection's epilogue
        ys = ws.moe_ys[:pairs]
        if rows_form:
            order = offs = slot = None
        elif route is not None:
            order, offs, slot = route["order"], route["off"], route["slot"]
        else:
            order, offs, slot = ws.moe_order, ws.moe_off, ws.moe_slot
            ops.moe_sort(ids, pairs, E, ws.moe_cnt, offs, order, slot)
        if not rows_form and ws.moe_xs is not None and ops.tc_usable(a, a.shape[1]) and f.ff % 8 == 0:
            xs = ws.moe_xs[:pairs]                  # tensor-core tiles fetch contiguous rows: put the tokens' rows in sorted order first
            ops.moe_gather(a, top, order, pairs, xs)
            ops.moe_linear(xs, 0, L["w_eup"], ids, order, offs, pairs, kind, mid, *act_args)
        else:
            ops.moe_linear(a, top, L["w_eup"], ids, order, offs, pairs, kind, mid, *act_args)
        ops.moe_linear(mid, 0, L["w_edown"], ids, order, offs, pairs, ops.ACT_NONE, ys)
        sh = None
        if shared_done is not None:
            torch.cuda.current_stream(self.dev).wait_event(shared_done)
            sh = ws.moe_sh[:T]
        elif f.shared_ff:
            sh = self._shared_expert(L, f, ws, T, a)
        gate_z = z[:, E] if gated_shared and z is not None else None
        if f.identity:
            ops.moe_combine_ex(ys, wts, slot, ids, f.experts, x_id, T, top, sh, gate_z, y)
        else:
            ops.moe_combine(ys, wts, slot, T, top, sh, gate_z, y)

    def _shared_expert(self, L, f: "MoeFfSpec", ws: _Workspace, T: int, a: torch.Tensor) -> torch.Tensor:
        smid = ws.ff_inner.view(-1)[:T * f.shared_ff].view(T, f.shared_ff)
        self._proj_act(ws.ff_proj, T, a, L["w_sup"], seqops.ACT_KINDS[f.act], smid, f.shared_limit, f.alpha, f.up_shift)
        sh = ws.moe_sh[:T]
        seqops.linear(smid, L["w_sdown"], sh)
        return sh
