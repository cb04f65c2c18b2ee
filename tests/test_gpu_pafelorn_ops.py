"""The operators the Pafelorn design added to libb200seq, each alone, against the plain float64 restatement in tests/pafelorn_oracle.py:
the bigram embedding with its carried previous token, the branch sum + output norm + residual, PolyNorm, soft caps, the general
attention prep (biases, weighted q / k norms per head and over the whole projection, both rotary pairings, band scaling of the
frequencies), attention with sink and head temperature, with soft cap and kept first tokens, with fewer value heads than key heads
(the two maps of differential attention), keys that stand out just inside and just outside every edge (window, kept tokens, page
border, far away among hundreds), the two gated recurrences over portions and reused slots, the soft-max router with correction and
identity experts."""
import math

import numpy as np
import pytest
import torch

import pafelorn_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    from blazr_b200 import seqops
    seqops.lib()
    return seqops


def dev_step(ops, entries, block_size=16, tokens=None):
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


def bf(t):
    return t.to(torch.bfloat16).to(torch.float32)


# ---- embedding ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("W,buckets", [(44, 7), (260, 1000)])
def test_bigram_embedding_over_portions(ops, W, buckets):
    """two sequences fed in portions (one of two tokens, single tokens): the previous token comes from the same portion or from the entry's
    carried value; position 0 reads the table's last row whatever the carried value says"""
    V, scale, mp, mc = 50, 1.7, 13, 7
    w = {"embed": bf(rnd(V, W, seed=1)), "bigram": bf(rnd(buckets + 1, W, seed=2))}
    emb = {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}
    seqs = {"a": torch.randint(0, V, (9,), generator=torch.Generator().manual_seed(3)).tolist(), "b": torch.randint(0, V, (5,), generator=torch.Generator().manual_seed(4)).tolist()}
    ref = {n: O.embed(s, {k: v.double() for k, v in w.items()}, emb) for n, s in seqs.items()}
    table, big = w["embed"].to(torch.bfloat16).to(DEV), w["bigram"].to(torch.bfloat16).to(DEV)
    fed = {"a": 0, "b": 0}
    for step in [[("a", 2), ("b", 1)], [("b", 1), ("a", 1)], [("a", 6), ("b", 3)]]:
        st, keep = dev_step(ops, [(k, fed[n], 0, pages_for(fed[n] + k)) for n, k in step])
        ids = torch.tensor([t for n, k in step for t in seqs[n][fed[n]:fed[n] + k]], dtype=torch.int32, device=DEV)
        prev = torch.tensor([seqs[n][fed[n] - 1] if fed[n] else 49 for n, k in step], dtype=torch.int32, device=DEV)
        T = ids.numel()
        x, a = torch.empty(T, W, device=DEV), torch.empty(T, W, device=DEV, dtype=torch.bfloat16)
        ops.embed_bigram(table, big, ids, prev, st, scale, buckets, mp, mc, x, a)
        o = 0
        for n, k in step:
            close(x[o:o + k], ref[n][fed[n]:fed[n] + k], 1e-6)
            close(a[o:o + k].float(), ref[n][fed[n]:fed[n] + k], 1e-2)
            o += k
            fed[n] += k
    x2 = torch.empty(T, W, device=DEV)
    ops.embed_bigram(table, None, ids, prev, st, scale, 0, 0, 0, x2, None)      # no bigram table: the plain scaled embedding
    close(x2, torch.cat([w["embed"][seqs[n][fed[n] - k:fed[n]]] for n, k in step]).double() * scale, 1e-6)


# ---- branch sum + output norm + residual ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("W", [44, 33, 1024, 4100])
def test_branch_norm_forms(ops, W):
    T, eps = 7, 1e-4
    x, y1, y2 = rnd(T, W, seed=1), rnd(T, W, seed=2, scale=3.0), rnd(T, W, seed=3, scale=0.2)
    w, b1, w1, w2, fw = 1 + rnd(W, seed=4, scale=0.2), rnd(W, seed=5), 1 + rnd(W, seed=6, scale=0.3), 1 + rnd(W, seed=7, scale=0.3), 1 + rnd(W, seed=8, scale=0.2)
    d = lambda t: t.to(DEV)
    X, Y1, Y2 = x.double(), y1.double(), y2.double()
    # one branch
    xo, ao = torch.empty(T, W, device=DEV), torch.empty(T, W, device=DEV)
    ops.branch_norm(d(x), d(y1), d(w), eps, x_out=xo, a_out=ao)
    ref = X + O.rms_norm(Y1, eps, w.double())
    close(xo, ref, 2e-6)
    close(ao, ref, 2e-6)
    # two scaled branches, a bias on the first
    ops.branch_norm(d(x), d(y1), d(w), eps, bias1=d(b1), s1=0.8, y2=d(y2), s2=0.9, x_out=xo, a_out=ao)
    close(xo, X + O.rms_norm(0.8 * (Y1 + b1.double()) + 0.9 * Y2, eps, w.double()), 2e-6)
    # two branches with norms of their own; only some rows, with the final norm behind
    rows = torch.tensor([5, 0, 6], dtype=torch.int32, device=DEV)
    fin = torch.empty(3, W, device=DEV)
    ops.branch_norm(d(x), d(y1), d(w), eps, w_b1=d(w1), s1=0.5, y2=d(y2), w_b2=d(w2), s2=0.5, rows=rows, a_out=fin, fin_w=d(fw))
    ref = X + O.rms_norm(0.5 * (O.rms_norm(Y1, eps, w1.double()) + O.rms_norm(Y2, eps, w2.double())), eps, w.double())
    close(fin, O.rms_norm(ref, eps, fw.double())[[5, 0, 6]], 2e-6)


@pytest.mark.parametrize("F", [20, 336, 4100])
def test_polynorm_and_softcap(ops, F):
    T, eps = 5, 1e-5
    z = rnd(T, F + 3, seed=1, scale=1.5)
    coef = torch.tensor([0.7, -0.4, 0.25, 0.1])
    out = torch.empty(T, F, device=DEV)
    ops.polynorm(z.to(DEV)[:, :F], coef.to(DEV), eps, out)
    close(out, O.polynorm(z[:, :F].double(), coef.double(), eps), 3e-6)
    x = rnd(T, F, seed=2, scale=20.0).to(DEV)
    ref = 9.0 * torch.tanh(x.double().cpu() / 9.0)
    ops.softcap(x, 9.0)
    close(x, ref, 2e-6)


# ---- attention ---------------------------------------------------------------------------------------------------------------------
def run_attention(ops, q, k, v, *, scale, window, cuts, keep_first=0, softcap=0.0, temp=None, sink=None, page_shuffle=False):
    """q [T, H, D], k [T, G, D], v [T, Gv, V] already normed and rotated: fed in portions `cuts` through prep (which only stores) and attend"""
    T, H, D = q.shape
    G, Gv, V = k.shape[1], v.shape[1], v.shape[2]
    nb = -(-T // 16)
    pages = list(range(nb))
    if page_shuffle:
        pages = [(7 * p + 3) % (nb + 5) for p in range(nb + 5)][:nb]
        assert len(set(pages)) == nb
    kpool = torch.full((nb + 5, 16, G, D), 77.0, device=DEV)
    vpool = torch.full((nb + 5, 16, Gv, V), 77.0, device=DEV)
    sk = sink.to(DEV) if sink is not None else None
    tp = temp.to(DEV) if temp is not None else None
    d = ops.attn_desc(H, G, D, V, scale, gated=False, window=window, sink=sk, value_heads=Gv if Gv != G else 0, softcap=softcap, head_scale=tp, keep_first=keep_first)
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1).float()
    outs = []
    lo = 0
    for n in cuts:
        st, keep = dev_step(ops, [(n, lo, 0, pages[:-(-(lo + n) // 16)])])
        p = proj[lo:lo + n].contiguous().to(DEV)
        ops.attn_prep_ex(p, st, d, kpool, vpool)
        o = torch.empty(n, H * V, device=DEV)
        need = ops.attn_scratch_floats(n, 1, H, G, V, T)
        ops.attn_ex(p, st, d, kpool, vpool, o, torch.empty(max(need, 1), device=DEV))
        outs.append(o.cpu())
        lo += n
    assert lo == T
    return torch.cat(outs).view(T, H, V)


def standout(q, k, i, j, h, g, gain=6.0):
    """make key j the one query (i, h) looks at: k_j <- gain * q_i / |q_i| on key head g"""
    k[j, g] = gain * q[i, h] / q[i, h].norm()


@pytest.mark.parametrize("cuts", [[300], [255, 1, 1, 43], [100, 2, 61, 3, 134]])
def test_windowed_attention_with_sink_and_temperature_at_every_edge(ops, cuts):
    """window 141 over 300 positions in pages of 16: keys that stand out just inside and just outside the window of chosen queries (in prompts
    and in single-token steps), at page borders, and 140 positions back among hundreds; the sink takes a large share of some heads"""
    T, H, G, D, V, window = 300, 4, 2, 12, 20, 141
    q, k, v = rnd(T, H, D, seed=1), rnd(T, G, D, seed=2), rnd(T, G, V, seed=3)
    for n, (i, h) in enumerate([(299, 0), (256, 1), (255, 2), (200, 3), (160, 0), (141, 1), (140, 2)]):
        j = i - window + (1 if n % 2 == 0 else 0)      # just inside / just outside
        if j >= 0:
            standout(q, k, i, j, h, h // 2, 9.0)
    standout(q, k, 290, 288, 2, 1)
    sink, temp = torch.tensor([2.0, -1.0, 4.0, 0.0]), torch.tensor([1.3, 0.6, 1.0, 2.0])
    got = run_attention(ops, q, k, v, scale=0.4, window=window, cuts=cuts, temp=temp, sink=sink, page_shuffle=True)
    ref = O.masked_attention(q.double(), k.double(), v.double(), 0.4, window, temp=temp.double(), sink=sink.double())
    close(got, ref, 1e-5)
    no_sink = O.masked_attention(q.double(), k.double(), v.double(), 0.4, window, temp=temp.double())
    assert (no_sink - ref).abs().max() > 0.05      # the sink matters in this test


@pytest.mark.parametrize("cuts,keep", [([200], 6), ([150, 1, 1, 48], 6), ([64, 2, 134], 70), ([3, 197], 1)])
def test_soft_capped_attention_with_kept_first_tokens(ops, cuts, keep):
    """window 50 with kept first tokens: a query far away looks at kept token keep - 1 (seen) and at token `keep` (not seen unless inside the window);
    kept tokens that are also inside the window count once"""
    T, H, G, D, V, window = 200, 3, 3, 10, 7, 50
    q, k, v = rnd(T, H, D, seed=4), rnd(T, G, D, seed=5), rnd(T, G, V, seed=6)
    standout(q, k, 199, keep - 1, 0, 0, 9.0)
    standout(q, k, 180, keep, 1, 1, 9.0)
    standout(q, k, 151, 151 - window, 2, 2, 9.0)
    standout(q, k, keep + 2, 0, 0, 0, 9.0)
    got = run_attention(ops, q, k, v, scale=0.5, window=window, cuts=cuts, keep_first=keep, softcap=3.0)
    ref = O.masked_attention(q.double(), k.double(), v.double(), 0.5, window, keep_first=keep, softcap=3.0)
    close(got, ref, 1e-5)
    assert (O.masked_attention(q.double(), k.double(), v.double(), 0.5, window, keep_first=keep) - ref).abs().max() > 0.05


def test_attention_with_fewer_value_heads_than_key_heads(ops):
    """the two maps of differential attention as plain heads: 2 G key heads over G value heads; then the combination a1 - lambda a2"""
    T, H, G, D, V = 70, 6, 3, 8, 12
    q, k, v = rnd(T, 2 * H, D, seed=7), rnd(T, 2 * G, D, seed=8), rnd(T, G, V, seed=9)
    got = run_attention(ops, q, k, v, scale=0.3, window=33, cuts=[40, 1, 29])
    ref = O.masked_attention(q.double(), k.double(), v.double(), 0.3, 33)
    close(got, ref, 1e-5)
    lam, sc, eps = 0.37, 0.6, 1e-5
    out = torch.empty(T, H * V, device=DEV)
    ops.diff_combine(got.reshape(T, -1).to(DEV), H, G, V, lam, sc, eps, out)
    R = H // G
    r5 = ref.view(T, G, 2, R, V)       # the kernel's head order is [key group][map][head of the group]
    want = O.rms_norm(r5[:, :, 0] - lam * r5[:, :, 1], eps) * sc
    close(out.view(T, G, R, V), want, 1e-5)


@pytest.mark.parametrize("full,half,bias", [(False, True, True), (True, False, False), (False, False, True)])
def test_general_prep_norms_rotation_bias(ops, full, half, bias):
    """prep alone: what lands in the pool and in the query columns against bias + weighted RMS norm (per head or over the whole projection) + rotation"""
    T, H, G, D, V, eps = 37, 4, 2, 10, 6, 1e-3
    rot = {"dims": 6, "base": 50.0, "scaling": {"factor": 3.0, "low": 1.0, "high": 4.0, "original": 16}}
    from blazr_b200.layered import RotarySpec
    spec = RotarySpec(dims=6, base=50.0, layout="half" if half else "interleaved", bands=(3.0, 1.0, 4.0, 16))
    fr = torch.from_numpy(spec.table()[0])
    close(fr, torch.tensor(O.rotary_frequencies(rot)), 1e-6)
    width = H * D + G * D + G * V
    proj = rnd(T, width + 5, seed=10)
    b = rnd(width, seed=11) if bias else None
    qw, kw = (1 + rnd(H * D, seed=12, scale=0.3), 1 + rnd(G * D, seed=13, scale=0.3)) if full else (1 + rnd(D, seed=12, scale=0.3), 1 + rnd(D, seed=13, scale=0.3))
    keep = [fr.to(DEV), qw.to(DEV), kw.to(DEV), b.to(DEV) if bias else None]
    d = ops.attn_desc(H, G, D, V, 1.0, gated=False, qk_eps=eps, rot_freq=keep[0], q_norm_w=keep[1], k_norm_w=keep[2], norm_full=full, rot_half=half, in_bias=keep[3])
    kpool, vpool = torch.zeros(3, 16, G, D, device=DEV), torch.zeros(3, 16, G, V, device=DEV)
    pd = proj.to(DEV)
    st, _ = dev_step(ops, [(T, 0, 0, [2, 0, 1])])
    ops.attn_prep_ex(pd[:, :width + 5], st, d, kpool, vpool)
    P = proj[:, :width].double() + (b.double() if bias else 0.0)
    q, k, v = P[:, :H * D], P[:, H * D:H * D + G * D], P[:, H * D + G * D:]
    if full:
        q, k = O.rms_norm(q, eps, qw.double()).view(T, H, D), O.rms_norm(k, eps, kw.double()).view(T, G, D)
    else:
        q, k = O.rms_norm(q.view(T, H, D), eps, qw.double()), O.rms_norm(k.view(T, G, D), eps, kw.double())
    lay = "half" if half else "interleaved"
    q, k = O.rotate(q, rot, lay), O.rotate(k, rot, lay)
    close(pd[:, :H * D].view(T, H, D), q, 2e-6)
    order = torch.cat([kpool[2], kpool[0], kpool[1]])[:T]
    close(order, k, 2e-6)
    close(torch.cat([vpool[2], vpool[0], vpool[1]])[:T], v.view(T, G, V), 1e-6)


# ---- recurrences -------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("C", [13, 256, 1030])
def test_min_gru_over_portions_and_reused_slots(ops, C):
    """two sequences in portions of changing size in shared steps (one portion longer than a group of the chunked form, portions that end inside
    a warp's share of a group); the slots hold another sequence's state at the start"""
    W = 24
    w = {"z": bf(rnd(C, W, seed=1, scale=0.4)), "z.b": rnd(C, seed=2), "x": bf(rnd(C, W, seed=3, scale=0.5)), "x.b": rnd(C, seed=4), "g": bf(rnd(C, W, seed=5, scale=0.4)),
         "o": torch.eye(C)}
    ha, hb = bf(rnd(40 + 1200, W, seed=6)), bf(rnd(9, W, seed=7))
    wd = {k: v.double() for k, v in w.items()}
    ref = {"a": O.min_gru(ha.double(), wd, ""), "b": O.min_gru(hb.double(), wd, "")}
    state = torch.full((3, C), 5.0, device=DEV)
    bias = torch.cat([w["z.b"], w["x.b"], torch.zeros(C)]).to(DEV)
    Wst = torch.cat([w["z"], w["x"], w["g"]]).double()
    H = {"a": ha, "b": hb}
    fed, slot = {"a": 0, "b": 0}, {"a": 2, "b": 0}
    for step in [[("a", 17), ("b", 2)], [("b", 1), ("a", 1)], [("a", 2), ("b", 6)], [("a", 20)], [("a", 1135)], [("a", 33)], [("a", 32)]]:
        st, keep = dev_step(ops, [(k, fed[n], slot[n], pages_for(fed[n] + k)) for n, k in step])
        h = torch.cat([H[n][fed[n]:fed[n] + k] for n, k in step])
        proj = torch.cat([torch.zeros(h.shape[0], 3), (h.double() @ Wst.T).float()], 1).to(DEV)      # columns behind three unused ones
        bias3 = torch.cat([torch.zeros(3, device=DEV), bias])
        out = torch.empty(h.shape[0], C, device=DEV)
        ops.min_gru(proj, 3, 3 + C, 3 + 2 * C, bias3, state, st, C, out)
        o = 0
        for n, k in step:
            close(out[o:o + k], ref[n][fed[n]:fed[n] + k], 1e-5)
            o += k
            fed[n] += k


@pytest.mark.parametrize("C,blocks,taps", [(12, 1, 1), (36, 3, 4), (264, 2, 5)])
def test_rg_lru_chain_over_portions(ops, C, blocks, taps):
    """convolution with a biased input and carried tail -> per-block gate projections -> the recurrence, in portions down to two tokens"""
    W = 20
    bw = C // blocks
    w = {"y": bf(rnd(C, W, seed=1, scale=0.4)), "y.b": rnd(C, seed=2), "x": bf(rnd(C, W, seed=3, scale=0.5)), "x.b": rnd(C, seed=4), "conv": rnd(C, taps, seed=5, scale=0.5),
         "conv.b": rnd(C, seed=6, scale=0.2), "ra": bf(rnd(blocks, bw, bw, seed=7, scale=1 / math.sqrt(bw))), "ra.b": rnd(blocks, bw, seed=8), "ri": bf(rnd(blocks, bw, bw, seed=9, scale=1 / math.sqrt(bw))),
         "ri.b": rnd(blocks, bw, seed=10), "lam": rnd(C, seed=11) - 2.0, "o": torch.eye(C)}
    h = bf(rnd(61 + 600, W, seed=12))
    wd = {k: v.double() for k, v in w.items()}
    ref = O.rg_lru(h.double(), wd, "", {"width": C, "blocks": blocks})
    state, cstate = torch.full((2, C), 5.0, device=DEV), torch.full((2, max(taps - 1, 1), C), 5.0, device=DEV)
    Wst = torch.cat([w["y"], w["x"]]).double()
    bias = torch.cat([w["y.b"], w["x.b"]]).to(DEV)
    wg = torch.cat([w["ra"], w["ri"]], 1).to(torch.bfloat16).contiguous().to(DEV)
    gb = torch.cat([w["ra.b"], w["ri.b"]], 1).reshape(-1).contiguous().to(DEV)
    sp = torch.nn.functional.softplus(w["lam"].double()).float().to(DEV)
    lo = 0
    for n in [7, 2, 1, 1, 30, 2, 18, 530, 65, 5]:
        st, keep = dev_step(ops, [(n, lo, 1, pages_for(lo + n))])
        proj = (h[lo:lo + n].double() @ Wst.T).float().to(DEV)
        u, gates, out = torch.empty(n, C, device=DEV), torch.empty(n, 2 * C, device=DEV), torch.empty(n, C, device=DEV)
        ops.causal_conv_ex(proj[:, C:2 * C], bias[C:], w["conv"].to(DEV), w["conv.b"].to(DEV), cstate, st, 0, u)
        ops.head_linear(u, wg, gates, 2 * bw)
        ops.rg_lru(u, gates, gb, sp, 8.0, proj, 0, bias, state, st, blocks, out)
        close(out, ref[lo:lo + n], 2e-5)
        lo += n


# ---- router ------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("E,I,top,T", [(5, 2, 2, 9), (12, 4, 3, 150), (3, 0, 1, 40), (2, 3, 5, 33)])
def test_softmax_router_with_correction_and_identity_experts(ops, E, I, top, T):
    W = 24
    n_out = E + I
    z = rnd(T, n_out + 1, seed=1, scale=1.5)
    corr = rnd(n_out, seed=2, scale=0.3)
    ids, wts = torch.empty(T * top, dtype=torch.int32, device=DEV), torch.empty(T * top, device=DEV)
    ops.moe_route_ex(z.to(DEV)[:, :n_out], n_out, 1, 1, top, ops.ROUTE_SOFTMAX, corr.to(DEV), ids, wts, None)
    s = torch.softmax(z[:, :n_out].double(), -1)
    choice = s + corr.double()
    ids_c, wts_c = ids.cpu().view(T, top), wts.cpu().view(T, top)
    for t in range(T):
        want = sorted(range(n_out), key=lambda e: (-choice[t, e].item(), e))[:top]
        assert sorted(ids_c[t].tolist()) == sorted(want)
        tot = s[t, want].sum()
        for j in range(top):
            assert abs(wts_c[t, j].item() - (s[t, ids_c[t, j]] / tot).item()) < 1e-5
    # combination: real experts' rows from ys, identity experts return the token's own input
    ys, x = rnd(T * top, W, seed=3).to(DEV), rnd(T, W, seed=4).to(DEV)
    sh = rnd(T, W, seed=5).to(DEV)
    y = torch.empty(T, W, device=DEV)
    zd = z.to(DEV)
    ops.moe_combine_ex(ys, wts, None, ids, E, x, T, top, sh, zd[:, n_out], y)
    ref = torch.sigmoid(z[:, n_out].double())[:, None] * sh.double().cpu()
    for t in range(T):
        for j in range(top):
            e = int(ids_c[t, j])
            ref[t] += wts_c[t, j].double() * (x[t].double().cpu() if e >= E else ys[t * top + j].double().cpu())
    close(y, ref, 1e-5)
