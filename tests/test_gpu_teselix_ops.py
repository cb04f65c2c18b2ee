"""The operators the Teselix design added to libb200seq, each alone, against the plain float64 restatement in
tests/teselix_oracle.py: token shift and the gated post-norm (with the carried shift state), rotary positions in both pairings,
retention in its single-token and chunked forms (portions, reused slots, a far memory), the latent-attention prep and the
attention with a sink over latent rows (scattered and reused pages, a far key among hundreds), per-head projections, the expert
table and gated experts."""
import math

import numpy as np
import pytest
import torch

import teselix_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    from blazr_b200 import seqops
    seqops.lib()
    return seqops


def dev_step(ops, entries, block_size=16):
    """entries: [(n_tokens, pos0, slot, block_table)] -> (StepDesc, keep-alive tensors)"""
    from blazr_b200.batch import StepEntry, build_step
    sa = build_step([StepEntry([0] * n, p0, slot, bt) for n, p0, slot, bt in entries], block_size)
    t = {k: torch.from_numpy(np.ascontiguousarray(getattr(sa, k))).to(DEV) for k in ("tok_ent", "tok_pos", "ent_start", "ent_slot", "ent_pos0", "block_table")}
    d = ops.StepDesc(t["tok_ent"].data_ptr(), t["tok_pos"].data_ptr(), t["ent_start"].data_ptr(), t["ent_slot"].data_ptr(), t["ent_pos0"].data_ptr(),
                     t["block_table"].data_ptr(), sa.T, sa.B, sa.block_table.shape[1], block_size)
    return d, t


def pages_for(n, block_size=16, first=0):
    return list(range(first, first + -(-n // block_size)))


def close(got, ref, tol):
    ref = ref.double()
    err = (got.double().cpu() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-30)
    assert err < tol, f"relative error {err:.3e} >= {tol}"


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


# ---- token shift and post-norm ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("W", [44, 33, 1024, 4100])
def test_token_shift_and_gated_post_norm_over_portions(ops, W):
    """two sequences in portions (one of them of two tokens, one a single token) that share the step; slots hold another sequence's
    leftovers at the start; the state is written by the post-norm of the mixer's sublayer, read by the shift of the next portion"""
    eps, alpha = 1e-4, 2.5
    xa, xb = rnd(11, W, seed=1) + 0.3, rnd(6, W, seed=2)
    mu = torch.rand(W, generator=torch.Generator().manual_seed(3))
    state = torch.full((3, W), 9.0, device=DEV)
    ya, yb, za, zb = rnd(11, W, seed=4), rnd(6, W, seed=5), rnd(11, W + 3, seed=6), rnd(6, W + 3, seed=7)
    gb, w, b = rnd(W, seed=8, scale=0.3), 1 + rnd(W, seed=9, scale=0.2), rnd(W, seed=10, scale=0.2)
    plan = [[("a", 5), ("b", 2)], [("b", 1), ("a", 2)], [("a", 4), ("b", 3)]]
    fed = {"a": 0, "b": 0}
    X, Y, Z, slot = {"a": xa, "b": xb}, {"a": ya, "b": yb}, {"a": za, "b": zb}, {"a": 2, "b": 0}
    for step in plan:
        st, keep = dev_step(ops, [(k, fed[n], slot[n], pages_for(fed[n] + k)) for n, k in step])
        x = torch.cat([X[n][fed[n]:fed[n] + k] for n, k in step]).to(DEV)
        y = torch.cat([Y[n][fed[n]:fed[n] + k] for n, k in step]).to(DEV)
        z = torch.cat([Z[n][fed[n]:fed[n] + k] for n, k in step]).to(DEV)
        T = x.shape[0]
        plain, shifted = torch.empty(T, W, device=DEV), torch.empty(T, W, device=DEV)
        ops.token_shift(x, mu.to(DEV), state, st, plain, shifted)
        xo, ao = torch.empty(T, W, device=DEV), torch.empty(T, W, device=DEV, dtype=torch.bfloat16)
        ops.post_norm(x, w.to(DEV), b.to(DEV), eps, y=y, zg=z[:, :W], gate_b=gb.to(DEV), alpha=alpha, x_out=xo, a_out=ao, state_out=state, step=st)
        o = 0
        for n, k in step:
            lo = fed[n]
            ref_shift = O.token_shift(X[n].double(), mu.double())[lo:lo + k]
            close(shifted[o:o + k], ref_shift, 1e-6)
            close(plain[o:o + k], X[n][lo:lo + k], 1e-7)
            v = alpha * X[n][lo:lo + k].double() + torch.sigmoid(Z[n][lo:lo + k, :W].double() + gb.double()) * Y[n][lo:lo + k].double()
            ref = O.layer_norm(v, w.double(), b.double(), eps)
            close(xo[o:o + k], ref, 1e-5)
            close(ao[o:o + k].float(), ref, 6e-3)
            o += k
            fed[n] += k
    assert ops.error_flags() == 0


def test_post_norm_with_the_next_shift_in_single_token_steps(ops):
    """single-token steps: the norm's kernel also forms the next mixer's shifted input from that mixer's own state"""
    W, eps = 40, 1e-5
    seq = rnd(7, W, seed=11)
    y = rnd(7, W, seed=12)
    w, b, mu = 1 + rnd(W, seed=13, scale=0.1), rnd(W, seed=14, scale=0.1), torch.rand(W, generator=torch.Generator().manual_seed(15))
    normed = O.layer_norm(1.5 * seq.double() + y.double(), w.double(), b.double(), eps)
    ref_shift = O.token_shift(normed, mu.double())
    next_state = torch.full((2, W), -4.0, device=DEV)
    for i in range(7):
        st, keep = dev_step(ops, [(1, i, 1, pages_for(i + 1))])
        xo, ao, sh = torch.empty(1, W, device=DEV), torch.empty(1, W, device=DEV), torch.empty(1, W, device=DEV)
        ops.post_norm(seq[i:i + 1].to(DEV), w.to(DEV), b.to(DEV), eps, y=y[i:i + 1].to(DEV), alpha=1.5, x_out=xo, a_out=ao, next_mu=mu.to(DEV), next_state=next_state,
                      a_shift_out=sh, step=st)
        close(xo, normed[i:i + 1], 1e-5)
        close(sh, ref_shift[i:i + 1], 1e-5)
        next_state[1] = xo[0]          # what the next layer's own post-norm would store: its input


def test_final_norm_gathers_rows(ops):
    W = 52
    x, w, b = rnd(9, W, seed=16), 1 + rnd(W, seed=17, scale=0.1), rnd(W, seed=18)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    out = torch.empty(3, W, device=DEV)
    ops.post_norm(x.to(DEV), w.to(DEV), b.to(DEV), 1e-6, rows=rows.to(DEV), a_out=out)
    close(out, O.layer_norm(x.double()[rows.long()], w.double(), b.double(), 1e-6), 1e-5)


# ---- rotary -----------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("layout,D,dims,scaling", [("half", 16, 16, None), ("half", 12, 6, None), ("interleaved", 10, 4, {"factor": 3.0, "original": 64, "fast": 8.0, "slow": 1.5}),
                                                  ("interleaved", 8, 8, None), ("half", 7, 2, None)])
def test_rotary_in_both_pairings(ops, layout, D, dims, scaling):
    from blazr_b200.layered import RotarySpec
    rot = {"dims": dims, "base": 500.0}
    if scaling:
        rot["scaling"] = scaling
    H, T, p0 = 3, 9, 37
    x = rnd(T, 5 + H * D + 2, seed=19)
    ref = O.rotate(torch.cat([torch.zeros(p0, H, D, dtype=torch.float64), x[:, 5:5 + H * D].double().reshape(T, H, D)]), rot, layout)[p0:] * 0.25
    fr, amp = RotarySpec(dims, 500.0, tuple(scaling[k] for k in ("factor", "original", "fast", "slow")) if scaling else None, layout).table()
    st, keep = dev_step(ops, [(T, p0, 0, pages_for(p0 + T))])
    xd = x.to(DEV)
    ops.rotary(xd, 5, H, D, st, torch.from_numpy(fr).to(DEV), layout == "half", amp, 0.25)
    close(xd[:, 5:5 + H * D].reshape(T, H, D), ref, 2e-6)
    assert torch.equal(xd[:, :5].cpu(), x[:, :5]) and torch.equal(xd[:, 5 + H * D:].cpu(), x[:, 5 + H * D:])


# ---- retention ------------------------------------------------------------------------------------------------------------------------------
def retention_reference(proj, H, D, V, decay, eps, rot):
    T = proj.shape[0]
    p = proj.double()
    q, k = p[:, :H * D].view(T, H, D), p[:, H * D:2 * H * D].view(T, H, D)
    v, g = p[:, 2 * H * D:2 * H * D + H * V].view(T, H, V), p[:, 2 * H * D + H * V:]
    q, k = O.rotate(q, rot, "half"), O.rotate(k, rot, "half") * D ** -0.5
    o = O.unit_rms(O.retention_scan(q, k, v, decay), eps).reshape(T, H * V)
    return o * g * torch.sigmoid(g)


def make_retention(ops, H, D, V, decay, eps, rot):
    from blazr_b200.layered import RotarySpec
    dec = torch.tensor([decay, [math.log2(d) for d in decay]], dtype=torch.float64).float().to(DEV)
    fr = torch.from_numpy(RotarySpec(rot["dims"], rot["base"], None, "half").table()[0]).to(DEV) if rot else None
    return ops.retention_desc(H, D, V, dec, eps, D ** -0.5, rot_freq=fr, rot_half=True), (dec, fr)


@pytest.mark.parametrize("H,D,V,rot", [(2, 8, 12, {"dims": 4, "base": 50.0}), (1, 80, 72, {"dims": 80, "base": 1e4}), (3, 6, 5, None), (2, 64, 64, {"dims": 64, "base": 1e6})])
def test_retention_portions_single_tokens_and_reused_slots(ops, H, D, V, rot):
    """two sequences over portions of 1, 2, 63, 64, 65 and 130 tokens and single-token steps, in slots that hold a finished sequence's
    state; every cut gives the whole-sequence result"""
    eps = 1e-5
    decay = [0.9, 0.9995, 0.97][:H]
    desc, keep0 = make_retention(ops, H, D, V, decay, eps, rot)
    n_in = 2 * H * D + 2 * H * V
    pa, pb = rnd(330, n_in, seed=21), rnd(140, n_in, seed=22)
    ra, rb = retention_reference(pa, H, D, V, decay, eps, rot), retention_reference(pb, H, D, V, decay, eps, rot)
    state = torch.full((3, H, D, V), 3.0, device=DEV)
    plan = [[("a", 1)], [("a", 2), ("b", 65)], [("a", 63), ("b", 1)], [("a", 1), ("b", 1)], [("a", 64), ("b", 2)], [("b", 1)], [("a", 130), ("b", 70)], [("a", 1)], [("a", 68)]]
    fed, P, R, slot = {"a": 0, "b": 0}, {"a": pa, "b": pb}, {"a": ra, "b": rb}, {"a": 1, "b": 2}
    for step in plan:
        st, keep = dev_step(ops, [(k, fed[n], slot[n], pages_for(fed[n] + k)) for n, k in step])
        proj = torch.cat([P[n][fed[n]:fed[n] + k] for n, k in step]).to(DEV)
        T = proj.shape[0]
        out = torch.empty(T, H * V, device=DEV)
        need = ops.retention_scratch_floats(T, len(step), H, D, V)
        assert (need == 0) == (T == len(step))
        scratch = torch.empty(max(need, 1), device=DEV)
        ops.retention(proj, st, desc, state, out, scratch)
        o = 0
        for n, k in step:
            close(out[o:o + k], R[n][fed[n]:fed[n] + k], 2e-5)
            o += k
            fed[n] += k
    assert fed == {"a": 330, "b": 140}


def test_retention_remembers_a_far_token(ops):
    """decay close to one: a key / value pair 700 tokens back, made large and met by a query that points at it, carries the output; a state
    that is lost, a decay applied once too often per chunk or a chunk's start state left out would all show"""
    H, D, V, eps = 1, 16, 8, 1e-6
    decay = [0.9999]
    desc, keep0 = make_retention(ops, H, D, V, decay, eps, None)
    n_in = 2 * H * D + 2 * H * V
    T = 760
    proj = rnd(T, n_in, seed=23, scale=0.05)
    key = torch.zeros(D)
    key[3] = 30.0
    proj[40, D:2 * D] = key
    proj[40, 2 * D:2 * D + V] = torch.arange(1, V + 1).float() * 5
    proj[745:, :D] = key * 0.5
    proj[:, 2 * D + V:] = 1.0
    ref = retention_reference(proj, H, D, V, decay, eps, None)
    assert (ref[750, :V] / ref[750, :V].norm() @ (torch.arange(1, V + 1).double() / torch.arange(1, V + 1).double().norm())).item() > 0.99
    state = torch.zeros(1, H, D, V, device=DEV)
    st, keep = dev_step(ops, [(700, 0, 0, pages_for(700))])
    out = torch.empty(700, H * V, device=DEV)
    ops.retention(proj[:700].to(DEV).clone(), st, desc, state, out, torch.empty(ops.retention_scratch_floats(700, 1, H, D, V), device=DEV))
    close(out, ref[:700], 2e-5)
    st, keep = dev_step(ops, [(50, 700, 0, pages_for(750))])
    out = torch.empty(50, H * V, device=DEV)
    ops.retention(proj[700:750].to(DEV).clone(), st, desc, state, out, torch.empty(ops.retention_scratch_floats(50, 1, H, D, V), device=DEV))
    close(out, ref[700:750], 2e-5)
    for i in range(750, T):
        st, keep = dev_step(ops, [(1, i, 0, pages_for(i + 1))])
        out = torch.empty(1, H * V, device=DEV)
        ops.retention(proj[i:i + 1].to(DEV).clone(), st, desc, state, out, None)
        close(out, ref[i:i + 1], 2e-5)


# ---- latent attention ---------------------------------------------------------------------------------------------------------------------
def latent_reference(kv, q, uk, uv, norm_w, sink, gate, H, Dn, Rd, V, R, scale, eps, rot):
    """kv [T, R + Rd], q [T, H * (Dn + Rd)] of one whole sequence -> gated head outputs [T, H * V]"""
    T = kv.shape[0]
    kv, q = kv.double(), q.double().view(T, H, Dn + Rd)
    c = O.unit_rms(kv[:, :R], eps) * norm_w.double()
    kr = O.rotate(kv[:, None, R:], rot, "interleaved")
    qr = O.rotate(q[:, :, Dn:], rot, "interleaved")
    kn, val = (c @ uk.double().T).view(T, H, Dn), (c @ uv.double().T).view(T, H, V)
    o = O.sink_softmax_attention(torch.cat([q[:, :, :Dn], qr], -1), torch.cat([kn, kr.expand(T, H, Rd)], -1), val, scale, sink.double())
    return (o * torch.sigmoid(gate.double())[:, :, None]).reshape(T, H * V)


def run_latent(ops, kv, q, gate, uk, uv, norm_w, sink, H, Dn, Rd, V, R, scale, eps, rot, plan, pages, kpool, act=torch.float32, expanded=False):
    """plan: steps of [(name, n)]; kv / q / gate: name -> whole-sequence tensors; pages: name -> block table; returns name -> [T, H * V].
    expanded: steps that are not all single tokens gather their contexts' latents, project per-head keys | values and attend over those"""
    from blazr_b200.layered import RotarySpec
    fr, amp = RotarySpec(Rd, rot["base"], None, "interleaved").table()
    fr = torch.from_numpy(fr).to(DEV)
    desc = ops.latent_attn_desc(H, R, Rd, scale, gated=True, sink=sink)
    ukT = uk.view(H, Dn, R).transpose(1, 2).contiguous().bfloat16().to(DEV)
    uvh = uv.view(H, V, R).contiguous().bfloat16().to(DEV)
    fed = {n: 0 for n in kv}
    outs = {n: [] for n in kv}
    for step in plan:
        st, keep = dev_step(ops, [(k, fed[n], 0, pages[n]) for n, k in step])
        T = sum(k for _, k in step)
        proj = torch.cat([torch.cat([kv[n][fed[n]:fed[n] + k], gate[n][fed[n]:fed[n] + k]], 1) for n, k in step]).to(DEV)
        qq = torch.cat([q[n][fed[n]:fed[n] + k] for n, k in step]).to(DEV)
        if expanded and T > len(step):
            ops.latent_prep(proj, 0, -1, qq, st, H, Dn, Rd, R, norm_w.to(DEV), eps, fr, amp, kpool, None, None)
            ctx = sum(fed[n] + k for n, k in step)
            cx, kvx = torch.empty(ctx, R, device=DEV, dtype=act), torch.empty(ctx, H * (Dn + V), device=DEV)
            ops.latent_gather(kpool, st, R, ctx, cx)
            ops.linear(cx, torch.cat([uk, uv]).bfloat16().to(DEV), kvx)
            dx = ops.expanded_attn_desc(H, Dn, Rd, V, scale, kpool.view(-1, R + Rd)[:, R:], gated=True, sink=sink)
            up = torch.empty(T, H * V, device=DEV, dtype=act)
            scratch = torch.empty(max(1, ops.attn_scratch_floats(T, len(step), H, H, V, 1024)), device=DEV)
            ops.attn_ex(qq, st, dx, kvx, kvx[:, H * Dn:], up, scratch, gate=proj[:, R + Rd:])
            o0 = 0
            for n, k in step:
                outs[n].append(up[o0:o0 + k].float().cpu())
                o0 += k
                fed[n] += k
            continue
        Qp = torch.zeros(T, H * (R + Rd), device=DEV)
        qn = torch.empty(T, H * Dn, device=DEV, dtype=act)
        ops.latent_prep(proj, 0, -1, qq, st, H, Dn, Rd, R, norm_w.to(DEV), eps, fr, amp, kpool, Qp, qn)
        ops.head_linear(qn, ukT, Qp, R + Rd)
        o = torch.empty(T, H * R, device=DEV, dtype=act)
        scratch = torch.empty(max(1, ops.attn_scratch_floats(T, len(step), H, 1, R, 1024)), device=DEV)
        ops.attn_ex(Qp, st, desc, kpool, None, o, scratch, gate=proj[:, R + Rd:])
        up = torch.empty(T, H * V, device=DEV, dtype=act)
        ops.head_linear(o, uvh, up, V, ops.ACT_IDENT)
        o0 = 0
        for n, k in step:
            outs[n].append(up[o0:o0 + k].float().cpu())
            o0 += k
            fed[n] += k
    return {n: torch.cat(v) for n, v in outs.items()}


@pytest.mark.parametrize("H,Dn,Rd,V,R", [(3, 5, 2, 7, 9), (4, 8, 8, 8, 16), (2, 16, 4, 12, 24)])
def test_latent_attention_over_scattered_and_reused_pages(ops, H, Dn, Rd, V, R):
    """two sequences in portions and single tokens over pages in shuffled order; a third sequence then takes over the first one's pages"""
    eps, scale, rot = 1e-5, 0.35, {"dims": Rd, "base": 200.0}
    mk = lambda n, s: (rnd(n, R + Rd, seed=s), rnd(n, H * (Dn + Rd), seed=s + 1), rnd(n, H, seed=s + 2))
    uk, uv = rnd(H * Dn, R, seed=30, scale=R ** -0.5).bfloat16().float(), rnd(H * V, R, seed=31, scale=R ** -0.5).bfloat16().float()
    norm_w, sink = 1 + rnd(R, seed=32, scale=0.1), rnd(H, seed=33, scale=1.5).to(DEV)
    seqs = {"a": mk(90, 40), "b": mk(37, 50), "c": mk(70, 60)}
    kpool = torch.full((16, 16, R + Rd), 50.0, device=DEV)
    perm = torch.randperm(16, generator=torch.Generator().manual_seed(34)).tolist()
    pages = {"a": perm[:6], "b": perm[6:9], "c": perm[:5]}
    ref = {n: latent_reference(kv, q, uk, uv, norm_w, sink.cpu(), g, H, Dn, Rd, V, R, scale, eps, rot) for n, (kv, q, g) in seqs.items()}
    plan = [[("a", 20), ("b", 1)], [("b", 2), ("a", 1)], [("a", 47), ("b", 30)], [("a", 1), ("b", 1)], [("a", 21), ("b", 3)], [("c", 2)], [("c", 67)], [("c", 1)]]
    for expanded in (False, True):      # in the latent space throughout; per-head keys for the steps with portions
        kpool.fill_(50.0)
        got = run_latent(ops, {n: s[0] for n, s in seqs.items()}, {n: s[1] for n, s in seqs.items()}, {n: s[2] for n, s in seqs.items()}, uk, uv, norm_w, sink, H, Dn, Rd, V, R,
                         scale, eps, rot, plan, pages, kpool, expanded=expanded)
        for n in seqs:
            close(got[n], ref[n], 2e-5)
    assert ops.error_flags() == 0


def test_latent_attention_finds_a_far_key_and_counts_the_sink_once(ops):
    """600 positions; the query of the last tokens points at the latent of position 7 (scaled so that its score stands out) - decoded alone
    (keys split among blocks) and inside a portion; a large sink then takes most of the weight, once, whatever the split"""
    H, Dn, Rd, V, R, eps, scale = 2, 8, 4, 8, 8, 1e-6, 1.0
    rot = {"dims": Rd, "base": 1e4}
    T = 600
    kv, q, gate = rnd(T, R + Rd, seed=70, scale=0.3), rnd(T, H * (Dn + Rd), seed=71, scale=0.3), torch.zeros(T, H) + 8.0
    uk = torch.eye(Dn, R).repeat(H, 1)            # the unrotated key of every head is the latent itself
    uv = torch.eye(V, R).repeat(H, 1)
    kv[7, :R] = torch.tensor([9.0, -9.0, 9.0, -9.0, 9.0, -9.0, 9.0, -9.0])
    norm_w = torch.ones(R)
    c7 = O.unit_rms(kv[7:8, :R].double(), eps)[0]
    for t in range(590, T):
        q[t].view(H, Dn + Rd)[:, :Dn] = c7.float() * 6.0
    for sink_value in (-20.0, 49.0):
        sink = torch.full((H,), sink_value, device=DEV)
        ref = latent_reference(kv, q, uk, uv, norm_w, sink.cpu(), gate, H, Dn, Rd, V, R, scale, eps, rot)
        if sink_value < 0:       # the far latent carries the output
            assert (ref[595, :V] / ref[595, :V].norm() @ c7 / c7.norm()).item() > 0.98
        else:                    # the sink (49) outweighs the far key (score about 6 * 8 = 48) but not by much
            assert 0.02 < ref[595, :V].norm().item() / c7.norm().item() < 0.9
        kpool = torch.zeros(40, 16, R + Rd, device=DEV)
        plan = [[("a", 580)], [("a", 13)]] + [[("a", 1)]] * 7
        for expanded in (False, True):
            got = run_latent(ops, {"a": kv}, {"a": q}, {"a": gate}, uk, uv, norm_w, sink, H, Dn, Rd, V, R, scale, eps, rot, plan, {"a": list(range(39, 1, -1))}, kpool,
                             expanded=expanded)
            close(got["a"][580:], ref[580:], 3e-5)
            close(got["a"][:580], ref[:580], 3e-5)


def test_latent_attention_with_a_wide_latent(ops):
    """a latent wider than 256: single tokens stay in the latent space (one query row per thread, 32 value columns each), portions attend over per-head keys"""
    H, Dn, Rd, V, R, eps, scale, rot = 3, 16, 8, 24, 320, 1e-5, 0.2, {"dims": 8, "base": 1000.0}
    kv, q, gate = rnd(60, R + Rd, seed=87), rnd(60, H * (Dn + Rd), seed=88), rnd(60, H, seed=89)
    uk, uv = rnd(H * Dn, R, seed=83, scale=R ** -0.5).bfloat16().float(), rnd(H * V, R, seed=84, scale=R ** -0.5).bfloat16().float()
    norm_w, sink = 1 + rnd(R, seed=85, scale=0.1), rnd(H, seed=86).to(DEV)
    ref = latent_reference(kv, q, uk, uv, norm_w, sink.cpu(), gate, H, Dn, Rd, V, R, scale, eps, rot)
    got = run_latent(ops, {"a": kv}, {"a": q}, {"a": gate}, uk, uv, norm_w, sink, H, Dn, Rd, V, R, scale, eps, rot, [[("a", 40)], [("a", 1)], [("a", 1)], [("a", 9)]] + [[("a", 1)]] * 9,
                     {"a": pages_for(60)}, torch.zeros(4, 16, R + Rd, device=DEV), expanded=True)
    close(got["a"], ref, 2e-5)


def test_bfloat16_activations_in_latent_attention(ops):
    H, Dn, Rd, V, R, eps, scale, rot = 4, 16, 8, 16, 32, 1e-5, 0.2, {"dims": 8, "base": 100.0}
    kv, q, gate = rnd(80, R + Rd, seed=80), rnd(80, H * (Dn + Rd), seed=81), rnd(80, H, seed=82)
    uk, uv = rnd(H * Dn, R, seed=83, scale=R ** -0.5).bfloat16().float(), rnd(H * V, R, seed=84, scale=R ** -0.5).bfloat16().float()
    norm_w, sink = 1 + rnd(R, seed=85, scale=0.1), rnd(H, seed=86).to(DEV)
    ref = latent_reference(kv, q, uk, uv, norm_w, sink.cpu(), gate, H, Dn, Rd, V, R, scale, eps, rot)
    for expanded in (False, True):
        got = run_latent(ops, {"a": kv}, {"a": q}, {"a": gate}, uk, uv, norm_w, sink, H, Dn, Rd, V, R, scale, eps, rot, [[("a", 70)]] + [[("a", 1)]] * 10, {"a": pages_for(80)},
                         torch.zeros(8, 16, R + Rd, device=DEV), act=torch.bfloat16, expanded=expanded)
        close(got["a"], ref, 3e-2)


# ---- experts ---------------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("T,E,top,ff,W,act", [(5, 4, 2, 10, 44, torch.float32), (90, 6, 3, 24, 48, torch.float32), (200, 8, 2, 32, 64, torch.bfloat16), (7, 3, 1, 8, 40, torch.bfloat16)])
def test_table_choice_and_gated_experts(ops, T, E, top, ff, W, act):
    """the experts of a token are the row of a table that its id picks, each weighted 1 / top; gated experts over per-pair rows (few pairs)
    and over sorted tiles (many pairs), plus a shared expert that is added as it is"""
    V, limit, sl = 29, 1.2, 0.8
    g = torch.Generator().manual_seed(90)
    table = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(V)]).to(torch.int32)
    tok = torch.randint(0, V, (T,), generator=g).to(torch.int32)
    x = rnd(T, W, seed=91).to(act)
    w = {"table": table}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"] = rnd(ff, W, seed=100 + e, scale=2 * W ** -0.5).bfloat16().double(), rnd(ff, W, seed=200 + e, scale=2 * W ** -0.5).bfloat16().double()
        w[f"e{e}.down"] = rnd(W, ff, seed=300 + e, scale=ff ** -0.5).bfloat16().double()
    w["shared.gate"], w["shared.up"], w["shared.down"] = (rnd(16, W, seed=401, scale=2 * W ** -0.5).bfloat16().double(), rnd(16, W, seed=402, scale=2 * W ** -0.5).bfloat16().double(),
                                                          rnd(W, 16, seed=403, scale=0.25).bfloat16().double())
    ref = O.table_experts(x.double(), tok.tolist(), w, "", {"router": {"top": top}, "expert": {"limit": limit}, "shared": {"limit": sl}})
    il = lambda a, b: torch.stack([a, b], 1).reshape(2 * a.shape[0], a.shape[1])
    w_up = torch.stack([il(w[f"e{e}.gate"], w[f"e{e}.up"]) for e in range(E)]).bfloat16().to(DEV)
    w_down = torch.stack([w[f"e{e}.down"] for e in range(E)]).bfloat16().to(DEV)
    pairs = T * top
    i32 = dict(dtype=torch.int32, device=DEV)
    ids, wts, cnt = torch.empty(pairs, **i32), torch.empty(pairs, device=DEV), torch.zeros(E, **i32)
    xd = x.to(DEV)
    ops.moe_table_route(table.to(DEV), tok.to(DEV), T, E, top, ids, wts, cnt)
    assert torch.equal(ids.cpu().view(T, top), table[tok.long()]) and bool((wts == 1.0 / top).all())
    assert torch.equal(cnt.cpu(), torch.bincount(table[tok.long()].flatten(), minlength=E).to(torch.int32))
    z2, mid, ys = torch.empty(pairs, 2 * ff, device=DEV), torch.empty(pairs, ff, device=DEV, dtype=act), torch.empty(pairs, W, device=DEV)
    mid2 = torch.empty(pairs, ff, device=DEV, dtype=act)
    if pairs <= 64:
        order = offs = slot = None
    else:
        order, offs, slot = torch.empty(pairs, **i32), torch.zeros(E + 1, **i32), torch.empty(pairs, **i32)
        ops.moe_sort(ids, pairs, E, cnt, offs, order, slot)
    ops.moe_linear(xd, top, w_up, ids, order, offs, pairs, ops.ACT_NONE, z2)               # product, then the activation ...
    ops.act(z2, ops.ACT_SWISH_CLAMP, mid2, limit, 1.702, 1.0)
    ops.moe_linear(xd, top, w_up, ids, order, offs, pairs, ops.ACT_SWISH_CLAMP, mid, limit, 1.702, 1.0)     # ... and both in one kernel
    close(mid.float(), mid2.float().cpu(), 1e-6 if act == torch.float32 else 1e-2)
    if order is not None and act == torch.bfloat16:      # rows in sorted order: the tensor-core tiles with the gated epilogue
        xs = torch.empty(pairs, W, device=DEV, dtype=act)
        ops.moe_gather(xd, top, order, pairs, xs)
        mid3 = torch.empty(pairs, ff, device=DEV, dtype=act)
        ops.moe_linear(xs, 0, w_up, ids, order, offs, pairs, ops.ACT_SWISH_CLAMP, mid3, limit, 1.702, 1.0)
        close(mid3.float(), mid2.float().cpu(), 2e-2)
    ops.moe_linear(mid, 0, w_down, ids, order, offs, pairs, ops.ACT_NONE, ys)
    smid, sh = torch.empty(T, 16, device=DEV, dtype=act), torch.empty(T, W, device=DEV)
    if T <= 8 or act == torch.bfloat16:
        ops.linear_act(xd, il(w["shared.gate"], w["shared.up"]).bfloat16().to(DEV), ops.ACT_SWISH_CLAMP, smid, sl, 1.702, 1.0)
    else:
        zs = torch.empty(T, 32, device=DEV)
        ops.linear(xd, il(w["shared.gate"], w["shared.up"]).bfloat16().to(DEV), zs)
        ops.act(zs, ops.ACT_SWISH_CLAMP, smid, sl, 1.702, 1.0)
    ops.linear(smid, w["shared.down"].bfloat16().to(DEV), sh)
    y = torch.empty(T, W, device=DEV)
    ops.moe_combine(ys, wts, slot, T, top, sh, None, y)
    close(y, ref, 2e-5 if act == torch.float32 else 2e-2)
    assert ops.error_flags() == 0


@pytest.mark.parametrize("T,H,N,K,xdt", [(3, 5, 7, 9, torch.float32), (2, 20, 16, 24, torch.bfloat16), (40, 3, 10, 6, torch.float32), (100, 4, 24, 16, torch.bfloat16),
                                         (300, 6, 136, 72, torch.bfloat16), (70, 2, 200, 64, torch.float32), (17, 4, 8, 8, torch.bfloat16)])
def test_per_head_projections(ops, T, H, N, K, xdt):
    """every head's slice of a row through that head's own weight: per-pair rows, exact tiles, tensor-core tiles per head; results at a pitch
    wider than N, columns between the heads' results untouched"""
    x = rnd(T, H * K + 8, seed=97).to(xdt)
    w = rnd(H, N, K, seed=98, scale=K ** -0.5).bfloat16()
    ref = torch.einsum("thk,hnk->thn", x[:, :H * K].double().view(T, H, K), w.double())
    pitch = N + 3
    out = torch.full((T, H * pitch + 2), 7.0, device=DEV)
    ops.head_linear(x.to(DEV)[:, :H * K], w.to(DEV), out, pitch)
    got = out[:, :H * pitch].view(T, H, pitch)
    close(got[:, :, :N], ref, 2e-6 if xdt == torch.float32 else 1e-5)
    assert bool((got[:, :, N:] == 7.0).all()) and bool((out[:, H * pitch:] == 7.0).all())
    ob = torch.empty(T, H * N, device=DEV, dtype=torch.bfloat16)
    ops.head_linear(x.to(DEV)[:, :H * K], w.to(DEV), ob, N, ops.ACT_IDENT)
    close(ob.float().view(T, H, N), ref, 6e-3)


def test_projection_written_in_the_activation_type(ops):
    """the identity kind: a product that feeds the next linear layer, on the weight-streaming rows, the per-pair rows and the tensor-core tiles"""
    for M, N, K in [(3, 24, 40), (70, 64, 96)]:
        x, w = rnd(M, K, seed=95).bfloat16(), rnd(N, K, seed=96, scale=K ** -0.5).bfloat16()
        out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        ops.linear_act(x.to(DEV), w.to(DEV), ops.ACT_IDENT, out)
        close(out.float(), x.double() @ w.double().T, 6e-3)
