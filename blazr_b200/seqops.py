"""Python harness over the C ABI of libb200seq.so (include/b200seq.h): dense bfloat16-weight linear layers and the sequence
operators of layer-list models (stream mixing + grouped RMS norm, carried-state causal convolutions, chunk / window attention
over a paged KV pool, the state-space recurrence, gated activations, the depth-averaged residual, mixtures of experts, retention,
latent attention, per-head projections, token shift + gated post-norm, the branch sum + output norm of two-branch mixers, the bigram
embedding, PolyNorm, soft caps, differential attention, minGRU and real-gated linear recurrences, soft-max routing with identity experts,
arg-max).

Like blazr_b200/ops.py, PyTorch is plumbing only (device memory, streams); every compute call goes through ctypes.  The library
is compiled on first use when it is missing (`ensure_built`): a fresh checkout needs nothing but nvcc.  There is no CPU
fallback: without the library or without an sm_100 GPU the calls raise.
"""
from __future__ import annotations

import ctypes as C
import fcntl
import os
import shutil
import subprocess
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
SRC_DIR = os.path.join(_HERE, "csrc", "seq")
LIB_PATH = os.environ.get("B200SEQ_LIB") or os.path.join(_HERE, "lib", "libb200seq.so")

F32, BF16 = 0, 2
CONV_RESIDUAL, CONV_SILU = 1, 2
ACT_SWISH_CLAMP, ACT_GELU_TANH, ACT_RELU2, ACT_IDENT = 0, 1, 2, 3   # gated: clamped swish, tanh-gelu gate; plain: squared relu, the product itself
ACT_NONE = -1
ACT_KINDS = {"swish_clamp": ACT_SWISH_CLAMP, "gelu_tanh": ACT_GELU_TANH, "relu2": ACT_RELU2}
ACT_GATED = (ACT_SWISH_CLAMP, ACT_GELU_TANH)
PATH_AUTO, PATH_ROWS, PATH_TILED, PATH_TC = 0, 1, 2, 3
TC_MIN_ROWS = 32   # b200seq_linear's automatic choice takes the tensor-core path from this many rows
_DT = {torch.float32: F32, torch.bfloat16: BF16}

EXPORTS = ["b200seq_last_error", "b200seq_version", "b200seq_launch_count", "b200seq_error_flags", "b200seq_embed_streams", "b200seq_hc_norm", "b200seq_hc_norm_conv",
           "b200seq_causal_conv", "b200seq_group_rmsnorm", "b200seq_gated_act", "b200seq_linear", "b200seq_linear_gated", "b200seq_attn_prep", "b200seq_attn", "b200seq_attn_scratch_floats",
           "b200seq_ssm_scan", "b200seq_ssm_scratch_floats", "b200seq_argmax", "b200seq_linear_act", "b200seq_act", "b200seq_depth_norm", "b200seq_attn_prep_ex",
           "b200seq_attn_ex", "b200seq_moe_route", "b200seq_moe_sort", "b200seq_moe_linear", "b200seq_moe_gather", "b200seq_moe_combine", "b200seq_moe_router", "b200seq_moe_table_route", "b200seq_moe_linear_act", "b200seq_head_linear", "b200seq_latent_gather",
           "b200seq_latent_prep", "b200seq_rotary", "b200seq_retention", "b200seq_retention_scratch_floats", "b200seq_token_shift", "b200seq_post_norm",
           "b200seq_moe_route_ex", "b200seq_moe_router_ex", "b200seq_moe_combine_ex", "b200seq_causal_conv_ex", "b200seq_embed_bigram", "b200seq_branch_norm", "b200seq_polynorm", "b200seq_softcap",
           "b200seq_diff_combine", "b200seq_min_gru", "b200seq_rg_lru"]


class SeqError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"b200seq error {code}: {msg}")
        self.code = code


class StepDesc(C.Structure):
    """b200seq_step: device pointers of one step's int32 arrays (see include/b200seq.h)"""
    _fields_ = [("tok_ent", C.c_void_p), ("tok_pos", C.c_void_p), ("ent_start", C.c_void_p), ("ent_slot", C.c_void_p), ("ent_pos0", C.c_void_p),
                ("block_table", C.c_void_p), ("T", C.c_int32), ("B", C.c_int32), ("max_blocks", C.c_int32), ("block_size", C.c_int32)]


class AttnDesc(C.Structure):
    """b200seq_attn_desc: sizes, columns of the projection row and mask / rotation constants of one attention layer"""
    _fields_ = [("H", C.c_int32), ("G", C.c_int32), ("D", C.c_int32), ("V", C.c_int32), ("q_col", C.c_int32), ("k_col", C.c_int32), ("v_col", C.c_int32),
                ("gate_col", C.c_int32), ("scale", C.c_float), ("chunk", C.c_int32), ("window", C.c_int32), ("pool", C.c_int32), ("qk_eps", C.c_float),
                ("rot_dims", C.c_int32), ("rot_freq", C.c_void_p), ("rot_scale", C.c_float), ("sink", C.c_void_p), ("latent_v", C.c_int32), ("gate", C.c_void_p), ("gate_ld", C.c_int64), ("ctx_rows", C.c_int32), ("kd", C.c_int32), ("kv_ld", C.c_int64), ("krot", C.c_void_p), ("krot_ld", C.c_int64),
                ("q_norm_w", C.c_void_p), ("k_norm_w", C.c_void_p), ("norm_full", C.c_int32), ("rot_half", C.c_int32), ("in_bias", C.c_void_p), ("kv_shared", C.c_int32),
                ("vg", C.c_int32), ("softcap", C.c_float), ("head_scale", C.c_void_p), ("keep_first", C.c_int32), ("gate_elem", C.c_int32)]


class RetentionDesc(C.Structure):
    """b200seq_retention_desc: sizes, columns of the projection row, decays and rotation constants of one retention layer"""
    _fields_ = [("H", C.c_int32), ("D", C.c_int32), ("V", C.c_int32), ("q_col", C.c_int32), ("k_col", C.c_int32), ("v_col", C.c_int32), ("g_col", C.c_int32),
                ("decay", C.c_void_p), ("eps", C.c_float), ("rot_dims", C.c_int32), ("rot_half", C.c_int32), ("rot_freq", C.c_void_p), ("rot_scale", C.c_float),
                ("k_scale", C.c_float)]


def retention_desc(H: int, D: int, V: int, decay: torch.Tensor, eps: float, k_scale: float, *, rot_freq: Optional[torch.Tensor] = None, rot_half: bool = True,
                   rot_scale: float = 1.0) -> "RetentionDesc":
    """descriptor for a projection row laid out q | k | v | gate; decay: device f32 [2, H] (decays, their base-2 logarithms); the caller
    keeps decay and rot_freq alive"""
    assert decay.dtype == torch.float32 and tuple(decay.shape) == (2, H) and decay.is_contiguous()
    d = RetentionDesc(H, D, V, 0, H * D, 2 * H * D, 2 * H * D + H * V, decay.data_ptr(), eps, 2 * rot_freq.numel() if rot_freq is not None else 0, int(rot_half),
                      rot_freq.data_ptr() if rot_freq is not None else None, rot_scale, k_scale)
    d.width = 2 * H * D + 2 * H * V
    return d


def attn_desc(H: int, G: int, D: int, V: int, scale: float, *, values_from_keys: bool = False, gated: bool = True, chunk: int = 0, window: int = 0, pool: int = 0,
              qk_eps: float = -1.0, rot_freq: Optional[torch.Tensor] = None, rot_scale: float = 1.0, sink: Optional[torch.Tensor] = None,
              q_norm_w: Optional[torch.Tensor] = None, k_norm_w: Optional[torch.Tensor] = None, norm_full: bool = False, rot_half: bool = False,
              in_bias: Optional[torch.Tensor] = None, kv_shared: bool = False, value_heads: int = 0, softcap: float = 0.0, head_scale: Optional[torch.Tensor] = None,
              keep_first: int = 0, gate_elem: bool = False) -> "AttnDesc":
    """descriptor for a projection row laid out q | k | v | gate (v absent when the values are the keys, k and v absent when they are another
    layer's (kv_shared), gate absent when not gated); value_heads: number of value heads when it is not G.
    Device tensors (rot_freq f32 [rot_dims / 2], sink / head_scale f32 [H], norm weights, in_bias f32 [row width]) are kept alive by the caller."""
    Gv = value_heads if value_heads > 0 else G
    k_col = H * D
    v_col = k_col if values_from_keys else k_col + G * D
    end = k_col if kv_shared else v_col + (G * D if values_from_keys else Gv * V)
    ptr = lambda t: t.data_ptr() if t is not None else None
    d = AttnDesc(H, G, D, V, 0, k_col, v_col, end if gated else -1, scale, chunk, window, pool, qk_eps, 2 * rot_freq.numel() if rot_freq is not None else 0,
                 ptr(rot_freq), rot_scale, ptr(sink), 0)
    d.q_norm_w, d.k_norm_w, d.norm_full, d.rot_half, d.in_bias = ptr(q_norm_w), ptr(k_norm_w), int(norm_full), int(rot_half), ptr(in_bias)
    d.kv_shared, d.vg, d.softcap, d.head_scale, d.keep_first = int(kv_shared), (Gv if Gv != G else 0), softcap, ptr(head_scale), keep_first
    d.gate_elem = int(gate_elem and gated)
    d.width = end + ((H * V if gate_elem else H) if gated else 0)
    return d


def expanded_attn_desc(H: int, Dn: int, Rd: int, V: int, scale: float, krot: torch.Tensor, *, gated: bool = True, sink: Optional[torch.Tensor] = None) -> "AttnDesc":
    """descriptor of the attend step of a latent-attention layer over per-head keys and values that were projected out of the step's gathered
    context: rows [H * Dn keys | H * V values]; the Rd rotated key dimensions of every head come from krot, a view [rows, Rd] of the paged pool"""
    D = Dn + Rd
    d = AttnDesc(H, H, D, V, 0, 0, H * Dn, 0 if gated else -1, scale, 0, 0, 0, -1.0, 0, None, 1.0, sink.data_ptr() if sink is not None else None, 0, None, 0,
                 1, Dn if Rd > 0 else 0, H * (Dn + V), krot.data_ptr() if Rd > 0 else None, krot.stride(-2) if Rd > 0 else 0)
    d.width = H * D
    return d


def latent_attn_desc(H: int, R: int, Rd: int, scale: float, *, gated: bool = True, sink: Optional[torch.Tensor] = None) -> "AttnDesc":
    """descriptor of the attend step of a latent-attention layer: H query heads of size R + Rd (latent-space query | rotated part) in rows
    [H * (R + Rd)] (gate logits: the `gate` argument of attn_ex) over ONE key head [c | kr] whose values are its first R floats; no rotation here (b200seq_latent_prep did it)"""
    D = R + Rd
    d = AttnDesc(H, 1, D, R, 0, 0, 0, 0 if gated else -1, scale, 0, 0, 0, -1.0, 0, None, 1.0, sink.data_ptr() if sink is not None else None, 1)
    d.width = H * D
    return d


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    srcs = [os.path.join(SRC_DIR, f) for f in os.listdir(SRC_DIR) if f.endswith((".cu", ".cuh"))] + [os.path.join(_HERE, "..", "include", "b200seq.h")]
    return any(os.path.getmtime(s) > t for s in srcs if os.path.exists(s))


def ensure_built(force: bool = False) -> str:
    """compile libb200seq.so (nvcc, sm_100a) if it is missing or older than its sources; safe against concurrent callers"""
    if "B200SEQ_LIB" in os.environ or not (force or _stale()):
        return LIB_PATH
    os.makedirs(os.path.dirname(LIB_PATH), exist_ok=True)
    with open(os.path.join(os.path.dirname(LIB_PATH), ".seq_build.lock"), "w") as lk:
        fcntl.flock(lk, fcntl.LOCK_EX)
        if force or _stale():
            env = dict(os.environ)
            if "NVCC" not in env and shutil.which("nvcc") is None:
                for cand in (os.path.join(env.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"), "/usr/local/cuda/bin/nvcc"):
                    if os.path.exists(cand):
                        env["NVCC"] = cand
                        break
            r = subprocess.run(["make", "-C", SRC_DIR, "-j8"], capture_output=True, text=True, env=env)
            if r.returncode != 0:
                raise SeqError(-3, "libb200seq build failed:\n" + r.stdout[-3000:] + r.stderr[-3000:])
    return LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        ensure_built()
        L = C.CDLL(LIB_PATH)
        L.b200seq_last_error.restype = C.c_char_p
        L.b200seq_launch_count.restype = C.c_int64
        _lib = L
    return _lib


def _check(rc: int):
    if rc != 0:
        raise SeqError(rc, lib().b200seq_last_error().decode())


def _st(t: torch.Tensor) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _p(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def launch_count() -> int:
    return int(lib().b200seq_launch_count())


def error_flags() -> int:
    f = C.c_int(0)
    _check(lib().b200seq_error_flags(C.byref(f)))
    return f.value


def _rows2d(t: torch.Tensor):
    assert t.dim() == 2 and t.stride(1) == 1, "row-major 2-D view expected"
    return t.shape[0], t.shape[1], t.stride(0)


# ---- per-operator timeline (bench / profiling aid): set `timeline = []` and every operator call appends
#      (name, shapes of its positional tensor arguments, positional scalars, start event, end event, keyword arguments as shapes /
#      scalars); None (default) costs nothing ------------------------------------------------------------------------------------
timeline = None


def _timed(fn):
    name = fn.__name__

    def wrap(*a, **k):
        tl = timeline
        if tl is None:
            return fn(*a, **k)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        r = fn(*a, **k)
        e1.record()
        shapes = tuple((tuple(t.shape), t.element_size()) if isinstance(t, torch.Tensor) else None for t in a)
        scal = tuple(t for t in a if isinstance(t, (int, float, bool)))
        kw = {n: ((tuple(t.shape), t.element_size()) if isinstance(t, torch.Tensor) else t) for n, t in k.items() if isinstance(t, (torch.Tensor, int, float, bool))}
        tl.append((name, shapes, scal, e0, e1, kw))
        return r

    wrap.__name__, wrap.__doc__ = name, fn.__doc__
    return wrap


# ---- operators (all arguments are device tensors; outputs are written in place) --------------------------------------------
@_timed
def embed_streams(table: torch.Tensor, ids: torch.Tensor, scale: float, X: torch.Tensor):
    T, S, W = X.shape
    _check(lib().b200seq_embed_streams(_p(table), _p(ids), C.c_float(scale), T, S, W, _p(X), _st(X)))


@_timed
def hc_norm(X: torch.Tensor, y: Optional[torch.Tensor], post: Optional[torch.Tensor], in_w: Optional[torch.Tensor], norm_w: Optional[torch.Tensor],
            groups: int, eps: float, out: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None):
    T, S, W = X.shape
    R = T if rows is None else rows.numel()
    _check(lib().b200seq_hc_norm(_p(X), _p(y), _p(post), _p(in_w), _p(norm_w), S, W, groups, C.c_float(eps), _p(rows), R, _p(out), _DT[out.dtype] if out is not None else F32, _st(X)))


@_timed
def hc_norm_conv(X: torch.Tensor, y: Optional[torch.Tensor], post: Optional[torch.Tensor], in_w: torch.Tensor, norm_w: torch.Tensor, groups: int, eps: float,
                 conv_w: torch.Tensor, conv_state: torch.Tensor, step: "StepDesc", out: torch.Tensor):
    """hc_norm followed by the residual carried convolution in one kernel; only for steps in which every entry brings one token"""
    T, S, W = X.shape
    _check(lib().b200seq_hc_norm_conv(_p(X), _p(y), _p(post), _p(in_w), _p(norm_w), S, W, groups, C.c_float(eps), _p(conv_w), _p(conv_state), C.byref(step),
                                      conv_w.shape[1], _p(out), _DT[out.dtype], _st(X)))


@_timed
def causal_conv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: Optional[torch.Tensor], step: "StepDesc", mode: int, out: torch.Tensor):
    T, Cn, ldx = _rows2d(x)
    _, _, ldo = _rows2d(out)
    _check(lib().b200seq_causal_conv(_p(x), C.c_int64(ldx), _p(w), _p(bias), _p(state), C.byref(step), Cn, w.shape[1], mode, _p(out), _DT[out.dtype],
                                     C.c_int64(ldo), _st(x)))


@_timed
def group_rmsnorm(x: torch.Tensor, w: Optional[torch.Tensor], groups: int, eps: float, out: torch.Tensor):
    T, D, ldx = _rows2d(x)
    assert out.is_contiguous()
    _check(lib().b200seq_group_rmsnorm(_p(x), C.c_int64(ldx), _p(w), T, D, groups, C.c_float(eps), _p(out), _DT[out.dtype], _st(x)))


@_timed
def gated_act(gu: torch.Tensor, limit: float, alpha: float, up_shift: float, out: torch.Tensor, interleaved: bool = False):
    T, F2, ldg = _rows2d(gu)
    assert out.is_contiguous() and out.shape[1] * 2 == F2
    _check(lib().b200seq_gated_act(_p(gu), C.c_int64(ldg), T, F2 // 2, C.c_float(limit), C.c_float(alpha), C.c_float(up_shift), int(interleaved), _p(out), _DT[out.dtype], _st(gu)))


@_timed
def linear(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, path: int = PATH_AUTO):
    """y[M, N] (f32) = x[M, K] . w[N, K]^T; w bf16 contiguous"""
    M, K, ldx = _rows2d(x)
    _, N, ldy = _rows2d(y)
    assert w.dtype == torch.bfloat16 and w.is_contiguous() and tuple(w.shape) == (N, K) and y.dtype == torch.float32 and y.shape[0] == M
    _check(lib().b200seq_linear(_p(x), _DT[x.dtype], C.c_int64(ldx), _p(w), M, N, K, _p(y), C.c_int64(ldy), path, _st(x)))


@_timed
def linear_gated(x: torch.Tensor, w_il: torch.Tensor, limit: float, alpha: float, up_shift: float, out: torch.Tensor):
    """out[M, F] = gated_act(x . w_il^T); w_il bf16 [2F, K] with alternating gate / up rows (up to 8 rows: any activation type;
    more: the tensor-core path, bf16 activations only)"""
    M, K, ldx = _rows2d(x)
    _, F, ldo = _rows2d(out)
    assert w_il.dtype == torch.bfloat16 and w_il.is_contiguous() and tuple(w_il.shape) == (2 * F, K) and out.shape[0] == M
    _check(lib().b200seq_linear_gated(_p(x), _DT[x.dtype], C.c_int64(ldx), _p(w_il), M, F, K, C.c_float(limit), C.c_float(alpha), C.c_float(up_shift), _p(out),
                                      _DT[out.dtype], C.c_int64(ldo), _st(x)))


@_timed
def linear_act(x: torch.Tensor, w: torch.Tensor, act: int, out: torch.Tensor, limit: float = 0.0, alpha: float = 0.0, shift: float = 0.0):
    """out = act(x . w^T) in one kernel; w bf16 [N, K]; gated kinds (rows of w alternate gate / up) give out [M, N / 2], plain kinds [M, N]
    (up to 8 rows: any activation type; more: the tensor-core path, bf16 activations only)"""
    M, K, ldx = _rows2d(x)
    _, F, ldo = _rows2d(out)
    N = w.shape[0]
    assert w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[1] == K and out.shape[0] == M and F == (N // 2 if act in ACT_GATED else N)
    _check(lib().b200seq_linear_act(_p(x), _DT[x.dtype], C.c_int64(ldx), _p(w), M, N, K, act, C.c_float(limit), C.c_float(alpha), C.c_float(shift), _p(out),
                                    _DT[out.dtype], C.c_int64(ldo), _st(x)))


@_timed
def act(z: torch.Tensor, kind: int, out: torch.Tensor, limit: float = 0.0, alpha: float = 0.0, shift: float = 0.0):
    """the same activation on a product that is in memory (z f32 [T, N]; gated kinds read interleaved pairs)"""
    T, N, ldz = _rows2d(z)
    _, _, ldo = _rows2d(out)
    _check(lib().b200seq_act(_p(z), C.c_int64(ldz), T, N, kind, C.c_float(limit), C.c_float(alpha), C.c_float(shift), _p(out), _DT[out.dtype], C.c_int64(ldo), _st(z)))


@_timed
def depth_norm(x_cur: torch.Tensor, out1: Optional[torch.Tensor], w1: Optional[torch.Tensor], eps: float, *, out2: Optional[torch.Tensor] = None,
               w2: Optional[torch.Tensor] = None, y1: Optional[torch.Tensor] = None, y2: Optional[torch.Tensor] = None, hist: Optional[torch.Tensor] = None,
               n_prev: int = 0, dwa: Optional[torch.Tensor] = None, hist_out: Optional[torch.Tensor] = None, x_out: Optional[torch.Tensor] = None,
               rows: Optional[torch.Tensor] = None):
    """residual sum of a parallel layer (x_cur + (y1 + y2)), learned average over the results of all layers so far (hist [>= n_prev, cap, W] holds the
    earlier ones, dwa [n_prev + 1]), and up to two weighted layer norms of the outcome; rows: only these token rows (outputs are row-compact)"""
    W = x_cur.shape[-1]
    R = x_cur.shape[0] if rows is None else rows.numel()
    o = out1 if out1 is not None else out2
    _check(lib().b200seq_depth_norm(_p(hist), C.c_int64(hist.stride(0) if hist is not None else 0), n_prev, _p(dwa), _p(x_cur), _p(y1), _p(y2), _p(hist_out), _p(x_out), W,
                                    C.c_float(eps), _p(w1), _p(w2), _p(rows), R, _p(out1), _p(out2), _DT[o.dtype] if o is not None else F32, _st(x_cur)))


@_timed
def attn_prep_ex(proj: torch.Tensor, step: "StepDesc", d: "AttnDesc", kpool: Optional[torch.Tensor], vpool: Optional[torch.Tensor],
                 kpooled: Optional[torch.Tensor] = None, vpooled: Optional[torch.Tensor] = None):
    _, _, ld = _rows2d(proj)
    _check(lib().b200seq_attn_prep_ex(_p(proj), C.c_int64(ld), C.byref(step), C.byref(d), _p(kpool), _p(vpool), _p(kpooled), _p(vpooled), _st(proj)))


@_timed
def attn_ex(proj: torch.Tensor, step: "StepDesc", d: "AttnDesc", kpool: torch.Tensor, vpool: Optional[torch.Tensor], out: torch.Tensor,
            scratch: Optional[torch.Tensor] = None, kpooled: Optional[torch.Tensor] = None, vpooled: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None):
    """gate: f32 [T, H] view (row stride free) of the gate logits when they do not lie in the query rows (d.gate_col is then only a flag)"""
    _, _, ld = _rows2d(proj)
    if gate is not None:        # the descriptor of a call is a copy: the layer's own stays as it was
        d2 = AttnDesc.from_buffer_copy(d)
        d2.gate, d2.gate_ld = gate.data_ptr(), gate.stride(0)
        d = d2
    assert out.is_contiguous() and (scratch is None or (scratch.dtype == torch.float32 and scratch.is_contiguous()))
    _check(lib().b200seq_attn_ex(_p(proj), C.c_int64(ld), C.byref(step), C.byref(d), _p(kpool), _p(vpool), _p(kpooled), _p(vpooled), _p(out), _DT[out.dtype], _p(scratch),
                                 C.c_size_t(scratch.numel() if scratch is not None else 0), _st(proj)))


@_timed
def moe_route(z: torch.Tensor, E: int, groups: int, keep: int, top: int, ids: torch.Tensor, wts: torch.Tensor, counts: Optional[torch.Tensor]):
    """z f32 [T, >= E] router logits -> ids int32 [T, top], wts f32 [T, top], counts int32 [E]"""
    T, _, ldz = _rows2d(z)
    assert ids.dtype == torch.int32 and wts.dtype == torch.float32 and ids.is_contiguous() and wts.is_contiguous() and ids.numel() >= T * top
    _check(lib().b200seq_moe_route(_p(z), C.c_int64(ldz), T, E, groups, keep, top, _p(ids), _p(wts), _p(counts), _st(z)))


@_timed
def moe_router(x: torch.Tensor, w: torch.Tensor, E: int, groups: int, keep: int, top: int, z: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor):
    """router projection (all rows of the stacked weight, into z) and the choice among the first E, for at most 8 tokens, in one kernel"""
    T, K, ldx = _rows2d(x)
    _, NR, ldz = _rows2d(z)
    assert w.dtype == torch.bfloat16 and w.is_contiguous() and tuple(w.shape) == (NR, K) and z.dtype == torch.float32 and z.shape[0] == T
    _check(lib().b200seq_moe_router(_p(x), _DT[x.dtype], C.c_int64(ldx), _p(w), T, NR, K, E, groups, keep, top, _p(z), C.c_int64(ldz), _p(ids), _p(wts), _st(x)))


@_timed
def moe_table_route(table: torch.Tensor, tok_ids: torch.Tensor, T: int, E: int, top: int, ids: torch.Tensor, wts: torch.Tensor, counts: Optional[torch.Tensor]):
    """ids[t][j] = table[tok_ids[t]][j], wts = 1 / top: the experts of a token are a row of a table indexed by its token id"""
    assert table.dtype == torch.int32 and table.is_contiguous() and table.shape[1] == top and tok_ids.dtype == torch.int32 and ids.numel() >= T * top
    _check(lib().b200seq_moe_table_route(_p(table), _p(tok_ids), T, E, top, _p(ids), _p(wts), _p(counts), _st(table)))


@_timed
def moe_sort(ids: torch.Tensor, pairs: int, E: int, counts: torch.Tensor, offs: torch.Tensor, order: torch.Tensor, slot_of: torch.Tensor):
    _check(lib().b200seq_moe_sort(_p(ids), pairs, E, _p(counts), _p(offs), _p(order), _p(slot_of), _st(ids)))


@_timed
def moe_linear(x: torch.Tensor, x_div: int, w: torch.Tensor, ids: torch.Tensor, order: Optional[torch.Tensor], offs: Optional[torch.Tensor], pairs: int, act: int,
               out: torch.Tensor, limit: float = 0.0, alpha: float = 0.0, shift: float = 0.0):
    """one projection of every (token, choice) pair through its expert's weight; w bf16 [E, N, K]; out [pairs, N] (f32 when act is ACT_NONE);
    gated kinds: the rows of every expert's weight alternate (gate j, up j) and out is [pairs, N / 2]"""
    _, K, ldx = _rows2d(x)
    _, No, ldo = _rows2d(out)
    E, N = w.shape[0], w.shape[1]
    assert w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[2] == K and out.shape[0] >= pairs and No == (N // 2 if act in ACT_GATED else N)
    _check(lib().b200seq_moe_linear_act(_p(x), _DT[x.dtype], C.c_int64(ldx), x_div, _p(w), _p(ids), _p(order), _p(offs), pairs, E, N, K, act, C.c_float(limit),
                                        C.c_float(alpha), C.c_float(shift), _p(out), _DT[out.dtype], C.c_int64(ldo), _st(x)))


@_timed
def head_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, ocol: int, act: int = ACT_NONE):
    """out[t, h * ocol + n] = w[h, n] . x[t, h * K : (h + 1) * K] for every head: x [T, >= H * K] rows, w bf16 [H, N, K], out [T, >= (H - 1) * ocol + N] rows
    (f32 when act is ACT_NONE, else a plain kind - ACT_IDENT: the product itself - in out's type)"""
    T, _, ldx = _rows2d(x)
    _, _, ldo = _rows2d(out)
    H, N, K = w.shape
    assert w.dtype == torch.bfloat16 and w.is_contiguous() and out.shape[0] == T and (act != ACT_NONE or out.dtype == torch.float32)
    _check(lib().b200seq_head_linear(_p(x), _DT[x.dtype], C.c_int64(ldx), _p(w), T, H, N, K, act, _p(out), _DT[out.dtype], C.c_int64(ldo), C.c_int64(ocol), _st(x)))


@_timed
def moe_gather(x: torch.Tensor, x_div: int, order: torch.Tensor, pairs: int, out: torch.Tensor):
    """out[r] = x[order[r] // x_div]: the tokens' bf16 activations in the sorted order of their pairs"""
    _, K, ldx = _rows2d(x)
    _, _, ldo = _rows2d(out)
    assert x.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and out.shape[0] >= pairs and out.shape[1] == K
    _check(lib().b200seq_moe_gather(_p(x), C.c_int64(ldx), _p(order), x_div, pairs, K, _p(out), C.c_int64(ldo), _st(x)))


@_timed
def moe_combine(ys: torch.Tensor, wts: torch.Tensor, slot_of: Optional[torch.Tensor], T: int, top: int, shared: Optional[torch.Tensor], gate_z: Optional[torch.Tensor],
                y: torch.Tensor):
    W = y.shape[1]
    assert ys.is_contiguous() and y.is_contiguous() and (shared is None or shared.is_contiguous())
    _check(lib().b200seq_moe_combine(_p(ys), _p(wts), _p(slot_of), T, top, W, _p(shared), _p(gate_z), C.c_int64(gate_z.stride(0) if gate_z is not None else 0), _p(y), _st(y)))


def tc_usable(x: torch.Tensor, K: int) -> bool:
    """whether the tensor-core path takes this activation matrix (bf16, K % 8 == 0, rows 16-byte aligned)"""
    return x.dtype == torch.bfloat16 and K % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0


@_timed
def attn_prep(qkvg: torch.Tensor, step: "StepDesc", kpool: torch.Tensor, vpool: torch.Tensor, H: int, G: int, D: int, V: int, qk_eps: float):
    _, _, ld = _rows2d(qkvg)
    _check(lib().b200seq_attn_prep(_p(qkvg), C.c_int64(ld), C.byref(step), _p(kpool), _p(vpool), H, G, D, V, C.c_float(qk_eps), _st(qkvg)))


def attn_scratch_floats(T: int, B: int, H: int, G: int, V: int, max_keys: int) -> int:
    """floats of work area the key-split path wants for a step of T tokens (0: the step fills the GPU without splitting)"""
    f = lib().b200seq_attn_scratch_floats
    f.restype = C.c_size_t
    return int(f(T, B, H, G, V, max_keys))


@_timed
def attn(qkvg: torch.Tensor, step: "StepDesc", kpool: torch.Tensor, vpool: torch.Tensor, H: int, G: int, D: int, V: int, scale: float, chunk: int,
         window: int, gated: bool, out: torch.Tensor, scratch: Optional[torch.Tensor] = None):
    _, _, ld = _rows2d(qkvg)
    assert out.is_contiguous() and (scratch is None or (scratch.dtype == torch.float32 and scratch.is_contiguous()))
    _check(lib().b200seq_attn(_p(qkvg), C.c_int64(ld), C.byref(step), _p(kpool), _p(vpool), H, G, D, V, C.c_float(scale), chunk, window, int(gated),
                              _p(out), _DT[out.dtype], _p(scratch), C.c_size_t(scratch.numel() if scratch is not None else 0), _st(qkvg)))


@_timed
def latent_prep(proj: torch.Tensor, c_col: int, gate_col: int, q: torch.Tensor, step: "StepDesc", H: int, Dn: int, Rd: int, R: int, norm_w: torch.Tensor, eps: float,
                rot_freq: Optional[torch.Tensor], rot_scale: float, kpool: torch.Tensor, Qp: Optional[torch.Tensor], qn: Optional[torch.Tensor]):
    """Qp and qn None: the rotated part of every query head turns in place in q (the step attends over per-head keys)"""
    _, _, ldp = _rows2d(proj)
    _, _, ldq = _rows2d(q)
    ldQ = _rows2d(Qp)[2] if Qp is not None else 0
    assert (qn is None or qn.is_contiguous()) and kpool.is_contiguous() and kpool.shape[-1] == R + Rd
    _check(lib().b200seq_latent_prep(_p(proj), C.c_int64(ldp), c_col, gate_col, _p(q), C.c_int64(ldq), C.byref(step), H, Dn, Rd, R, _p(norm_w), C.c_float(eps),
                                     _p(rot_freq), C.c_float(rot_scale), _p(kpool), _p(Qp), C.c_int64(ldQ), _p(qn), _DT[qn.dtype] if qn is not None else F32, _st(proj)))


@_timed
def latent_gather(kpool: torch.Tensor, step: "StepDesc", R: int, ctx_rows: int, out: torch.Tensor):
    """out[r] = the latent (first R floats) of the r-th (entry, position) of the step's contexts, from the paged pool, in out's type"""
    assert kpool.is_contiguous() and out.is_contiguous() and out.shape[0] >= ctx_rows and out.shape[1] == R
    _check(lib().b200seq_latent_gather(_p(kpool), C.c_int64(kpool.shape[-1]), C.byref(step), R, ctx_rows, _p(out), _DT[out.dtype], _st(kpool)))


@_timed
def rotary(x: torch.Tensor, col: int, nheads: int, D: int, step: "StepDesc", rot_freq: Optional[torch.Tensor], half: bool, rot_scale: float = 1.0, mult: float = 1.0):
    _, _, ld = _rows2d(x)
    _check(lib().b200seq_rotary(_p(x), C.c_int64(ld), col, nheads, D, C.byref(step), 2 * rot_freq.numel() if rot_freq is not None else 0, int(half), _p(rot_freq),
                                C.c_float(rot_scale), C.c_float(mult), _st(x)))


def retention_scratch_floats(T: int, B: int, H: int, D: int, V: int) -> int:
    """floats of work area a retention step of T tokens in B entries wants (0: every entry brings one token)"""
    f = lib().b200seq_retention_scratch_floats
    f.restype = C.c_size_t
    return int(f(T, B, H, D, V))


@_timed
def retention(proj: torch.Tensor, step: "StepDesc", d: "RetentionDesc", state: torch.Tensor, out: torch.Tensor, scratch: Optional[torch.Tensor] = None):
    _, _, ld = _rows2d(proj)
    assert out.is_contiguous() and state.is_contiguous() and (scratch is None or (scratch.dtype == torch.float32 and scratch.is_contiguous()))
    _check(lib().b200seq_retention(_p(proj), C.c_int64(ld), C.byref(step), C.byref(d), _p(state), _p(out), _DT[out.dtype], _p(scratch),
                                   C.c_size_t(scratch.numel() if scratch is not None else 0), _st(proj)))


@_timed
def token_shift(x: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, step: "StepDesc", out_plain: Optional[torch.Tensor], out_shift: torch.Tensor):
    T, W = x.shape
    assert x.is_contiguous() and out_shift.is_contiguous() and (out_plain is None or (out_plain.is_contiguous() and out_plain.dtype == out_shift.dtype))
    _check(lib().b200seq_token_shift(_p(x), W, _p(mu), _p(state), C.byref(step), _p(out_plain), _p(out_shift), _DT[out_shift.dtype], _st(x)))


@_timed
def post_norm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float, *, y: Optional[torch.Tensor] = None, zg: Optional[torch.Tensor] = None,
              gate_b: Optional[torch.Tensor] = None, alpha: float = 1.0, rows: Optional[torch.Tensor] = None, x_out: Optional[torch.Tensor] = None,
              a_out: Optional[torch.Tensor] = None, state_out: Optional[torch.Tensor] = None, next_mu: Optional[torch.Tensor] = None,
              next_state: Optional[torch.Tensor] = None, a_shift_out: Optional[torch.Tensor] = None, step: Optional["StepDesc"] = None):
    """layer norm (weight, bias) after the gated residual sum: LN(alpha * x + sigmoid(zg + gate_b) * y); see include/b200seq.h"""
    W = x.shape[-1]
    R = x.shape[0] if rows is None else rows.numel()
    o = a_out if a_out is not None else a_shift_out
    assert x.is_contiguous() and (y is None or y.is_contiguous())
    _check(lib().b200seq_post_norm(_p(x), _p(y), _p(zg), C.c_int64(zg.stride(0) if zg is not None else 0), _p(gate_b), C.c_float(alpha), _p(w), _p(b), C.c_float(eps), W,
                                   _p(rows), R, _p(x_out), _p(a_out), _DT[o.dtype] if o is not None else F32, _p(state_out), _p(next_mu), _p(next_state), _p(a_shift_out),
                                   C.byref(step) if step is not None else None, _st(x)))


def ssm_scratch_floats(T: int, B: int, H: int, V: int, N: int) -> int:
    """floats of work area the segmented (parallel over time) scan wants for a step of T tokens in B entries; 0: none needed"""
    f = lib().b200seq_ssm_scratch_floats
    f.restype = C.c_size_t
    return int(f(T, B, H, V, N))


@_timed
def ssm_scan(proj: torch.Tensor, z0: int, dt0: int, xbc: torch.Tensor, A_log: torch.Tensor, Dp: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor,
             step: "StepDesc", H: int, V: int, N: int, G: int, out: torch.Tensor, scratch: Optional[torch.Tensor] = None):
    _, _, ldp = _rows2d(proj)
    _, _, ldx = _rows2d(xbc)
    assert out.is_contiguous() and (scratch is None or (scratch.dtype == torch.float32 and scratch.is_contiguous()))
    _check(lib().b200seq_ssm_scan(_p(proj), C.c_int64(ldp), z0, dt0, _p(xbc), C.c_int64(ldx), _p(A_log), _p(Dp), _p(dt_bias), _p(state), C.byref(step),
                                  H, V, N, G, _p(out), _p(scratch), C.c_size_t(scratch.numel() if scratch is not None else 0), _st(proj)))


@_timed
def argmax(logits: torch.Tensor, ids: torch.Tensor):
    R, V = logits.shape
    assert logits.is_contiguous() and ids.dtype == torch.int32
    _check(lib().b200seq_argmax(_p(logits), R, V, _p(ids), _st(logits)))


# ---- layers with the norm on the sublayer's output, two-branch mixers, gated linear recurrences ----------------------------------------------
ROUTE_SIGMOID, ROUTE_SOFTMAX = 0, 1


@_timed
def moe_route_ex(z: torch.Tensor, E: int, groups: int, keep: int, top: int, kind: int, correction: Optional[torch.Tensor], ids: torch.Tensor, wts: torch.Tensor,
                 counts: Optional[torch.Tensor]):
    """moe_route with the score kind (ROUTE_SIGMOID / ROUTE_SOFTMAX over the E logits) and a correction f32 [E] that enters the choice only"""
    T, _, ldz = _rows2d(z)
    assert ids.dtype == torch.int32 and wts.dtype == torch.float32 and ids.is_contiguous() and wts.is_contiguous() and ids.numel() >= T * top
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == E)
    _check(lib().b200seq_moe_route_ex(_p(z), C.c_int64(ldz), T, E, groups, keep, top, kind, _p(correction), _p(ids), _p(wts), _p(counts), _st(z)))


@_timed
def moe_router_ex(x: torch.Tensor, w: torch.Tensor, E: int, groups: int, keep: int, top: int, kind: int, correction: Optional[torch.Tensor], z: torch.Tensor,
                  ids: torch.Tensor, wts: torch.Tensor):
    """moe_router (projection and choice of at most 8 tokens in one kernel) with the score kind and correction of moe_route_ex"""
    T, K, ldx = _rows2d(x)
    _, NR, ldz = _rows2d(z)
    assert w.dtype == torch.bfloat16 and w.is_contiguous() and tuple(w.shape) == (NR, K) and z.dtype == torch.float32 and z.shape[0] == T
    _check(lib().b200seq_moe_router_ex(_p(x), _DT[x.dtype], C.c_int64(ldx), _p(w), T, NR, K, E, groups, keep, top, kind, _p(correction), _p(z), C.c_int64(ldz), _p(ids),
                                       _p(wts), _st(x)))


@_timed
def moe_combine_ex(ys: torch.Tensor, wts: torch.Tensor, slot_of: Optional[torch.Tensor], ids: torch.Tensor, E_real: int, x_id: torch.Tensor, T: int, top: int,
                   shared: Optional[torch.Tensor], gate_z: Optional[torch.Tensor], y: torch.Tensor):
    """moe_combine where a pair whose expert id is >= E_real is an identity expert: its output is the token's row of x_id (f32 [T, W])"""
    W = y.shape[1]
    assert ys.is_contiguous() and y.is_contiguous() and (shared is None or shared.is_contiguous()) and x_id.is_contiguous() and x_id.dtype == torch.float32
    _check(lib().b200seq_moe_combine_ex(_p(ys), _p(wts), _p(slot_of), _p(ids), E_real, _p(x_id), T, top, W, _p(shared), _p(gate_z),
                                        C.c_int64(gate_z.stride(0) if gate_z is not None else 0), _p(y), _st(y)))


@_timed
def causal_conv_ex(x: torch.Tensor, in_bias: Optional[torch.Tensor], w: torch.Tensor, bias: Optional[torch.Tensor], state: Optional[torch.Tensor], step: "StepDesc",
                   mode: int, out: torch.Tensor, out2: Optional[torch.Tensor] = None):
    """causal_conv over x + in_bias (mode 0: convolution + bias, nothing else); out2: a second copy of the result in its own type"""
    T, Cn, ldx = _rows2d(x)
    _, _, ldo = _rows2d(out)
    ldo2 = _rows2d(out2)[2] if out2 is not None else 0
    _check(lib().b200seq_causal_conv_ex(_p(x), C.c_int64(ldx), _p(in_bias), _p(w), _p(bias), _p(state), C.byref(step), Cn, w.shape[1], mode, _p(out), _DT[out.dtype],
                                        C.c_int64(ldo), _p(out2), _DT[out2.dtype] if out2 is not None else F32, C.c_int64(ldo2), _st(x)))


@_timed
def embed_bigram(table: torch.Tensor, bigram: Optional[torch.Tensor], ids: torch.Tensor, ent_prev: torch.Tensor, step: "StepDesc", scale: float, buckets: int,
                 mul_prev: int, mul_cur: int, x: torch.Tensor, a: Optional[torch.Tensor]):
    """x[t] = table[ids[t]] * scale + bigram[hash(previous token, token)] (the last row of bigram at position 0); a: the same in its own type"""
    W = x.shape[-1]
    assert table.dtype == torch.bfloat16 and table.is_contiguous() and x.is_contiguous() and x.dtype == torch.float32 and (a is None or a.is_contiguous())
    assert bigram is None or (bigram.dtype == torch.bfloat16 and bigram.is_contiguous() and tuple(bigram.shape) == (buckets + 1, W))
    _check(lib().b200seq_embed_bigram(_p(table), _p(bigram), _p(ids), _p(ent_prev), C.byref(step), C.c_float(scale), buckets, mul_prev, mul_cur, W, _p(x), _p(a),
                                      _DT[a.dtype] if a is not None else F32, _st(x)))


@_timed
def branch_norm(x: torch.Tensor, y1: torch.Tensor, w: torch.Tensor, eps: float, *, bias1: Optional[torch.Tensor] = None, w_b1: Optional[torch.Tensor] = None, s1: float = 1.0,
                y2: Optional[torch.Tensor] = None, w_b2: Optional[torch.Tensor] = None, s2: float = 1.0, rows: Optional[torch.Tensor] = None,
                x_out: Optional[torch.Tensor] = None, a_out: Optional[torch.Tensor] = None, fin_w: Optional[torch.Tensor] = None):
    """x + rms_norm(s1 * b1 + s2 * b2) * w with b1 = y1 + bias1 (rms-normed with w_b1 when given), b2 = y2 (rms-normed with w_b2); see include/b200seq.h"""
    W = x.shape[-1]
    R = x.shape[0] if rows is None else rows.numel()
    assert x.is_contiguous() and y1.is_contiguous() and (y2 is None or y2.is_contiguous()) and (a_out is None or a_out.is_contiguous())
    _check(lib().b200seq_branch_norm(_p(x), _p(y1), _p(bias1), _p(w_b1), C.c_float(s1), _p(y2), _p(w_b2), C.c_float(s2), _p(w), C.c_float(eps), W, _p(rows), R, _p(x_out),
                                     _p(a_out), _DT[a_out.dtype] if a_out is not None else F32, _p(fin_w), _st(x)))


@_timed
def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float, out: torch.Tensor):
    """out = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 per row, N = division by the root mean square; coef device f32 [4]"""
    T, F, ldz = _rows2d(z)
    _, _, ldo = _rows2d(out)
    assert coef.dtype == torch.float32 and coef.numel() == 4 and out.shape[1] == F
    _check(lib().b200seq_polynorm(_p(z), C.c_int64(ldz), T, F, _p(coef), C.c_float(eps), _p(out), _DT[out.dtype], C.c_int64(ldo), _st(z)))


@_timed
def softcap(x: torch.Tensor, cap: float):
    assert x.is_contiguous() and x.dtype == torch.float32
    _check(lib().b200seq_softcap(_p(x), C.c_int64(x.numel()), C.c_float(cap), _st(x)))


@_timed
def diff_combine(a: torch.Tensor, H: int, G: int, V: int, lam: float, out_scale: float, eps: float, out: torch.Tensor):
    """a f32 [T, 2 * H * V], the two maps per head in the order [key group][map][head of the group] -> out [T, H * V] = unit_rms(a1 - lam * a2) * out_scale"""
    T = a.shape[0]
    assert a.is_contiguous() and a.dtype == torch.float32 and a.shape[1] == 2 * H * V and out.is_contiguous() and tuple(out.shape) == (T, H * V)
    _check(lib().b200seq_diff_combine(_p(a), T, H, G, V, C.c_float(lam), C.c_float(out_scale), C.c_float(eps), _p(out), _DT[out.dtype], _st(a)))


@_timed
def min_gru(proj: torch.Tensor, z_col: int, x_col: int, g_col: int, bias: Optional[torch.Tensor], state: torch.Tensor, step: "StepDesc", Cn: int, out: torch.Tensor):
    _, _, ldp = _rows2d(proj)
    assert out.is_contiguous() and out.shape[1] == Cn and state.is_contiguous() and state.shape[1] == Cn
    _check(lib().b200seq_min_gru(_p(proj), C.c_int64(ldp), z_col, x_col, g_col, _p(bias), _p(state), C.byref(step), Cn, _p(out), _DT[out.dtype], _st(proj)))


@_timed
def rg_lru(u: torch.Tensor, gates: torch.Tensor, gate_bias: Optional[torch.Tensor], sp_lam: torch.Tensor, decay_c: float, proj: torch.Tensor, y_col: int,
           bias: Optional[torch.Tensor], state: torch.Tensor, step: "StepDesc", blocks: int, out: torch.Tensor):
    _, Cn, ldu = _rows2d(u)
    _, _, ldg = _rows2d(gates)
    _, _, ldp = _rows2d(proj)
    assert out.is_contiguous() and out.shape[1] == Cn and state.is_contiguous() and state.shape[1] == Cn and sp_lam.numel() == Cn
    _check(lib().b200seq_rg_lru(_p(u), C.c_int64(ldu), _p(gates), C.c_int64(ldg), _p(gate_bias), _p(sp_lam), C.c_float(decay_c), _p(proj), C.c_int64(ldp), y_col, _p(bias),
                                _p(state), C.byref(step), Cn, blocks, _p(out), _DT[out.dtype], _st(proj)))
