"""GPU: every mechanism of the post-norm hybrid decoder (Kenetar) alone, against the plain restatement in
oracle/kenetar_ref.py (fp64).  Sizes are awkward on purpose (odd widths, head sizes that are no multiple of a warp, a
vector or a page), and where random numbers would hide a fault the inputs are made so that it shows."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _ops():
    from vllm_neuron_b200 import ops

    return ops


def _meta(entries, blocks, bs=8):
    from vllm_neuron_b200.hybrid import StepMeta

    return StepMeta.build(entries, blocks, bs, DEV)


def _close(got, want, tol):
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).abs().max().item() / max(want.abs().max().item(), 1e-30)
    assert err < tol, err


def _pages(n, bs, first=1):
    return list(range(first, first + -(-n // bs)))


# ------------------------------------------------------------------------------------------------ embedding
def test_bigram_embedding_first_token_previous_token_state_and_slot_reuse():
    from oracle.kenetar_ref import embed_tokens

    ops = _ops()
    g = torch.Generator().manual_seed(0)
    V, W, buckets, mp, mc, scale = 61, 20, 13, 31, 7, 3.5
    Wt = {"embed": torch.randn(V, W, generator=g), "bigram": torch.randn(buckets + 1, W, generator=g)}
    e = {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}
    seqs = {0: torch.randint(0, V, (11,), generator=g).tolist(), 1: torch.randint(0, V, (5,), generator=g).tolist()}
    want = {s: embed_tokens(t, {k: v.double() for k, v in Wt.items()}, e) for s, t in seqs.items()}
    prev = torch.full((3,), 5, dtype=torch.int32, device=DEV)   # stale values: a fresh sequence must not read them
    table, big = Wt["embed"].to(DEV), Wt["bigram"].to(DEV)
    at = {0: 0, 1: 0}
    for step in ([(0, 3), (1, 1)], [(0, 1), (1, 2)], [(0, 1)], [(1, 2), (0, 6)]):      # slots: sequence 0 -> 2, sequence 1 -> 0
        entries = [({0: 2, 1: 0}[s], at[s], n) for s, n in step]
        toks = [t for s, n in step for t in seqs[s][at[s]:at[s] + n]]
        meta = _meta(entries, {2: [1, 2], 0: [3]})
        x, h = ops.embed_bigram(torch.tensor(toks, dtype=torch.int32, device=DEV), table, scale, meta, bigram=big, buckets=buckets,
                                mul_prev=mp, mul_cur=mc, prev_state=prev)
        ref = torch.cat([want[s][at[s]:at[s] + n] for s, n in step])
        _close(x, ref, 1e-6)
        _close(h, ref, 1e-6)
        for s, n in step:
            at[s] += n
    assert prev.tolist() == [seqs[1][-1], 5, seqs[0][-1]]
    # slot 2 goes to a NEW sequence: its first token takes the table's last row, not a row hashed from the old owner's token
    new = [7, 9]
    meta = _meta([(2, 0, 2)], {2: [4]})
    x, _ = ops.embed_bigram(torch.tensor(new, dtype=torch.int32, device=DEV), table, scale, meta, bigram=big, buckets=buckets,
                            mul_prev=mp, mul_cur=mc, prev_state=prev)
    _close(x, embed_tokens(new, {k: v.double() for k, v in Wt.items()}, e), 1e-6)
    # no bigram table: the scaled token row alone
    x, _ = ops.embed_bigram(torch.tensor(new, dtype=torch.int32, device=DEV), table, scale, meta)
    _close(x, Wt["embed"][new].double() * scale, 1e-6)


# ------------------------------------------------------------------------------------------------ norms and activations
def test_rms_residual_offset_weight_and_weighted_branch_sum():
    from oracle.kenetar_ref import offset_rms_norm

    ops = _ops()
    g = torch.Generator().manual_seed(1)
    T, W, top, eps = 6, 50, 3, 1e-3
    x, y, w = torch.randn(T, W, generator=g), torch.randn(T * top, W, generator=g) * 0.01, 0.2 * torch.randn(W, generator=g)
    wt = torch.rand(T, top, generator=g)
    for odt, tol in ((torch.float32, 1e-6), (torch.bfloat16, 5e-3)):
        xd = x.to(DEV).clone()
        h = ops.rms_residual(xd, y.to(DEV), w.to(DEV), eps, nsum=top, y_weight=wt.to(DEV), out_dtype=odt)
        s = (y.double().view(T, top, W) * wt.double()[:, :, None]).sum(1)
        want = x.double() + offset_rms_norm(s, w.double(), eps)
        _close(xd, want, 1e-6)                                  # the residual stream stays fp32 in both modes
        _close(h, want, tol)
    # eps sits inside the root (the branch here is small against it), and the weight is stored around zero
    plain = x.double() + s / s.pow(2).mean(-1, keepdim=True).sqrt() * w.double()
    assert (plain - want).abs().max() > 0.1
    xd = x.to(DEV).clone()
    assert ops.rms_residual(xd, y[:T].contiguous().to(DEV), w.to(DEV), eps) is None
    _close(xd, x.double() + offset_rms_norm(y[:T].double(), w.double(), eps), 1e-6)


def test_rmsnorm_over_a_column_range_and_per_head_gated_norm():
    from oracle.kenetar_ref import rms_unit

    ops = _ops()
    g = torch.Generator().manual_seed(2)
    T, eps = 5, 1e-4
    src, w = torch.randn(T, 77, generator=g), torch.randn(30, generator=g)
    _close(ops.rmsnorm_cols(src.to(DEV), 9, 30, w.to(DEV), eps, torch.float32), rms_unit(src[:, 9:39].double(), eps) * w, 2e-6)
    _close(ops.rmsnorm_cols(src.to(DEV), 9, 30, w.to(DEV), eps, torch.float32, offset=2.0),
           rms_unit(src[:, 9:39].double(), eps) * (2 + w.double()), 2e-6)
    H, P = 3, 21
    o, wn = torch.randn(T, H * P, generator=g), torch.randn(P, generator=g)
    gsrc = torch.randn(T, 10 + H * P, generator=g)
    gate = gsrc[:, 10:].double().view(T, H, P)
    want = rms_unit(o.double().view(T, H, P), eps) * wn * F.silu(gate)      # norm first, gate second; one weight for all heads
    _close(ops.head_rmsnorm_gate(o.to(DEV), gsrc.to(DEV), 10, wn.to(DEV), eps, H, torch.float32), want.reshape(T, H * P), 2e-6)
    wrong = rms_unit((o.double().view(T, H, P) * F.silu(gate)), eps) * wn
    assert (want - wrong).abs().max() > 0.05


def test_gated_units_silu_and_tanh_gelu():
    from oracle.kenetar_ref import gelu_tanh

    ops = _ops()
    g = torch.Generator().manual_seed(3)
    T, ff = 4, 37
    gu = torch.randn(T, 2 * ff, generator=g) * 3
    gate, up = gu[:, :ff].double(), gu[:, ff:].double()
    _close(ops.glu(gu.to(DEV), ops.ACT_GELU_TANH, torch.float32), gelu_tanh(gate) * up, 2e-6)
    _close(ops.glu(gu.to(DEV), ops.ACT_SILU, torch.float32), F.silu(gate) * up, 2e-6)
    assert (gelu_tanh(gate) - F.gelu(gate)).abs().max() > 1e-4              # the tanh form, not the erf form


# ------------------------------------------------------------------------------------------------ router and experts
@pytest.mark.parametrize("E,top", [(5, 1), (8, 3), (16, 16)])
def test_router_takes_the_largest_biased_logits_and_softmaxes_the_chosen_only(E, top):
    ops = _ops()
    g = torch.Generator().manual_seed(4)
    T = 40
    z = torch.randn(T, E, generator=g)
    bias = 2 * torch.randn(E, generator=g)                      # large enough to change the choice
    idx, wt = ops.moe_topk(z.to(DEV), top, bias=bias.to(DEV), mode=ops.ROUTE_SOFTMAX_TOP)
    val, want_idx = (z.double() + bias).topk(top, dim=-1)
    assert torch.equal(idx.cpu().long(), want_idx)
    _close(wt, torch.softmax(val, dim=-1), 1e-6)
    assert not torch.equal(want_idx, z.topk(top, dim=-1).indices) or top == E
    if top < E:                                                  # not the softmax over all experts
        assert (torch.softmax(z.double() + bias, -1).gather(1, want_idx) - wt.cpu().double()).abs().max() > 1e-3


@pytest.mark.parametrize("dtype,T", [(torch.float32, 9), (torch.bfloat16, 9), (torch.bfloat16, 400)])
def test_experts_weighted_on_their_outputs(dtype, T):
    from oracle.kenetar_ref import offset_rms_norm, softmax_topk_moe

    ops = _ops()
    g = torch.Generator().manual_seed(5)
    W, E, top, ff = 48, 4, 2, 24
    Wt = {"router": torch.randn(E, W, generator=g) * W ** -0.5, "router.b": torch.randn(E, generator=g)}
    for e in range(E):
        Wt.update({f"e{e}.gate": torch.randn(ff, W, generator=g) * W ** -0.5, f"e{e}.up": torch.randn(ff, W, generator=g) * W ** -0.5,
                   f"e{e}.down": torch.randn(W, ff, generator=g) * ff ** -0.5})
    Wt = {k: v.to(dtype).double() for k, v in Wt.items()}
    h = torch.randn(T, W, generator=g).to(dtype)
    want = softmax_topk_moe(h.double(), Wt, "", {"router": {"experts": E, "top": top}})
    dev = lambda t: t.to(DEV, dtype).contiguous()
    w_gu = dev(torch.stack([torch.cat([Wt[f"e{e}.gate"], Wt[f"e{e}.up"]]) for e in range(E)]))
    w_down = dev(torch.stack([Wt[f"e{e}.down"] for e in range(E)]))
    hd = h.to(DEV)
    logits = ops.linear_simt(hd, dev(Wt["router"]))
    idx, wt = ops.moe_topk(logits, top, bias=Wt["router.b"].float().to(DEV), mode=ops.ROUTE_SOFTMAX_TOP)
    align = ops.moe_align(idx, E, ops.moe_wide_tiles(hd, w_gu, idx.numel()))
    pairs = ops.moe_experts(hd, wt, align, w_gu, w_down, top, act=ops.ACT_SILU, scale_input=False)
    x = torch.zeros(T, W, device=DEV)
    ops.rms_residual(x, pairs, torch.zeros(W, device=DEV), 1e-6, nsum=top, y_weight=wt)
    ref = offset_rms_norm(want, torch.zeros(W).double(), 1e-6)
    got, ref = x.double().cpu(), ref
    if dtype == torch.float32:
        _close(got, ref, 1e-5)
    else:   # bf16 rounding of the hidden activations; a near-tie of the router may flip a row
        bad = ((got - ref).abs().amax(-1) > 0.05).float().mean().item()
        assert bad <= 0.02, bad


# ------------------------------------------------------------------------------------------------ gated delta rule
def _delta_reference(qc, kc, v, rb, ra, A_log, dt_bias, H, G, D, P):
    """qc / kc / v: convolved activations (fp64).  Unit vectors, beta, decay and the recurrence, per the restatement."""
    from oracle.kenetar_ref import gated_delta_rule

    T = qc.shape[0]
    unit = lambda a: a / torch.sqrt(a.pow(2).sum(-1, keepdim=True) + 1e-6)
    q = (unit(qc.view(T, G, D)) * D ** -0.5).repeat_interleave(H // G, dim=1)
    k = unit(kc.view(T, G, D)).repeat_interleave(H // G, dim=1)
    beta = torch.sigmoid(rb)
    gd = torch.exp(-torch.exp(A_log) * F.softplus(ra + dt_bias))
    return gated_delta_rule(q, k, v.view(T, H, P), beta, gd).reshape(T, H * P)


@pytest.mark.parametrize("H,G,D,P", [(4, 2, 12, 20), (3, 3, 32, 64), (2, 1, 100, 36), (2, 2, 300, 8), (1, 1, 5, 130), (2, 1, 600, 4)])
def test_delta_rule_portions_slots_and_sizes(H, G, D, P):
    """Two sequences advance in ragged portions (1, 2 and many tokens; a chunk of the kernel's staging is 16) through slots
    that held another sequence's state before; every step must continue the whole-sequence recurrence."""
    ops = _ops()
    g = torch.Generator().manual_seed(6)
    C = 2 * G * D + H * P
    n = {0: 75, 1: 23}
    data = {}
    for s, T in n.items():
        qkv = torch.randn(T, C, generator=g)
        proj = torch.randn(T, 5 + 2 * H, generator=g) * 2      # raw beta at column 5, raw decay input at 5 + H
        data[s] = (qkv, proj)
    A_log, dt_bias = torch.log(0.5 + torch.rand(H, generator=g)), torch.randn(H, generator=g)
    want = {}
    for s, (qkv, proj) in data.items():
        q, k, v = qkv.double().split([G * D, G * D, H * P], dim=-1)
        want[s] = _delta_reference(q, k, v, proj[:, 5:5 + H].double(), proj[:, 5 + H:].double(), A_log.double(), dt_bias.double(),
                                   H, G, D, P)
    state = torch.randn(4, H, P, D, device=DEV)                 # garbage: position 0 must not read it
    at = {0: 0, 1: 0}
    slot = {0: 3, 1: 1}
    sched = ([(0, 1), (1, 2)], [(0, 2), (1, 1)], [(0, 17)], [(0, 1), (1, 16)], [(0, 33), (1, 1)], [(1, 3), (0, 21)])
    for step in sched:
        entries = [(slot[s], at[s], c) for s, c in step]
        meta = _meta(entries, {3: list(range(1, 11)), 1: list(range(11, 14))})
        qkv = torch.cat([data[s][0][at[s]:at[s] + c] for s, c in step]).to(DEV).contiguous()
        proj = torch.cat([data[s][1][at[s]:at[s] + c] for s, c in step]).to(DEV).contiguous()
        o = ops.delta_rule(qkv, proj, 5, 5 + H, A_log.to(DEV), dt_bias.to(DEV), state, meta, H, G, D, P, D ** -0.5)
        ref = torch.cat([want[s][at[s]:at[s] + c] for s, c in step])
        _close(o, ref, 2e-5)
        for s, c in step:
            at[s] += c
    assert at == n


def test_delta_rule_write_is_visible_to_its_own_readout_and_decay_comes_first():
    """One head, hand-made numbers: with S = 0, o_1 = beta (k.q) v (the read-out sees the token's own write); the second
    token's prediction uses the DECAYED state."""
    ops = _ops()
    D, P = 4, 2
    k = torch.tensor([[1.0, 0, 0, 0], [1.0, 0, 0, 0]])
    q = torch.tensor([[2.0, 0, 0, 0], [2.0, 0, 0, 0]])
    v = torch.tensor([[3.0, -1.0], [5.0, 4.0]])
    qkv = torch.cat([q, k, v], dim=1).to(DEV).contiguous()
    proj = torch.tensor([[0.0, 0.3], [1.0, -0.2]], device=DEV)                   # raw beta, raw decay input
    A_log, dt_bias = torch.tensor([0.1], device=DEV), torch.tensor([0.2], device=DEV)
    state = torch.zeros(1, 1, P, D, device=DEV)
    o = ops.delta_rule(qkv, proj, 0, 1, A_log, dt_bias, state, _meta([(0, 0, 2)], {0: [1]}), 1, 1, D, P, D ** -0.5)
    b = torch.sigmoid(torch.tensor([0.0, 1.0]).double())
    gd = torch.exp(-math.exp(0.1) * F.softplus(torch.tensor([0.3, -0.2]).double() + 0.2))
    qs = 1.0 * D ** -0.5                                                          # unit q times dim^-1/2 (k is a unit vector already)
    s1 = b[0] * v[0].double()                                                     # row of S along k after token 1
    s2 = gd[1] * s1 + b[1] * (v[1].double() - gd[1] * s1)
    _close(o, torch.stack([s1 * qs, s2 * qs]), 1e-5)


# ------------------------------------------------------------------------------------------------ latent attention
def _rot(dims, scaling=True):
    return {"dims": dims, "base": 5000.0,
            "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0} if scaling else None}


@pytest.mark.parametrize("C,R,n", [(24, 16, 16), (40, 12, 8), (7, 6, 6)])
def test_latent_cache_rows_normed_latent_and_rotated_shared_key(C, R, n):
    from oracle.kenetar_ref import rms_unit, rotate_pairs, yarn_angles
    from vllm_neuron_b200.hybrid import RotSpec

    ops = _ops()
    g = torch.Generator().manual_seed(7)
    bs, T, eps = 8, 21, 1e-5
    rot = _rot(n)
    cos, sin = (t.to(DEV) for t in RotSpec(n, rot["base"], rot["scaling"]).tables(64))
    src, w = torch.randn(T, 3 + C + R, generator=g), torch.randn(C, generator=g)
    pos0 = 13                                                   # the portion crosses a page border at position 16
    pages = [5, 2, 9, 4, 7]
    meta = _meta([(1, pos0, T)], {1: pages}, bs)
    pool = torch.zeros(12, 1, bs, C + R, device=DEV)
    ops.latent_kv_write(src.to(DEV), 3, C, R, n, w.to(DEV), eps, cos, sin, meta, pool)
    c_ref = rms_unit(src[:, 3:3 + C].double(), eps) * w
    rc, rs = yarn_angles(rot, range(pos0, pos0 + T), torch.float64)
    kr = torch.cat([rotate_pairs(src[:, 3 + C:3 + C + n].double(), rc, rs), src[:, 3 + C + n:].double()], dim=-1)
    rows = torch.stack([pool[pages[p // bs], 0, p % bs] for p in range(pos0, pos0 + T)])
    _close(rows[:, :C], c_ref, 2e-6)
    _close(rows[:, C:], kr, 2e-6)
    # the query side turns by the same angles and keeps the unrotated part apart
    H, D = 3, 10
    q = torch.randn(T, H * (D + R), generator=g)
    nope, q_att = ops.latent_q_prep(q.to(DEV), H, D, R, n, C, cos, sin, meta, torch.float32)
    qv = q.double().view(T, H, D + R)
    _close(nope, qv[..., :D].reshape(T, H * D), 1e-7)
    qr = torch.cat([rotate_pairs(qv[..., D:D + n], rc, rs), qv[..., D + n:]], dim=-1)
    _close(q_att.view(T, H, C + R)[..., C:], qr, 2e-6)


def test_yarn_blend_differs_from_plain_and_from_fully_stretched_angles():
    from oracle.kenetar_ref import yarn_angles
    from vllm_neuron_b200.hybrid import RotSpec

    rot = _rot(16)
    cos, sin = RotSpec(16, rot["base"], rot["scaling"]).tables(300)
    rc, rs = yarn_angles(rot, range(300), torch.float64)
    assert (cos.double() - rc).abs().max() < 1e-6 and (sin.double() - rs).abs().max() < 1e-6
    pc, _ = yarn_angles(_rot(16, scaling=False), range(300), torch.float64)
    assert (rc - pc).abs().max() > 0.1                           # neither the unscaled angles ...
    f = rot["base"] ** (-2 * torch.arange(8, dtype=torch.float64) / 16) / 8.0
    sc = torch.cos(torch.arange(300, dtype=torch.float64)[:, None] * f) * (0.1 * math.log(8.0) + 1)
    assert (rc - sc).abs().max() > 0.1                           # ... nor every pair divided by the factor
    assert abs(rc[0, 0].item() - (0.1 * math.log(8.0) + 1)) < 1e-12


def _attend_latents(q_att, rows, scale, C, pos):
    """Plain softmax attention of one query over cache rows 0..pos: scores over the whole row, values = first C columns."""
    s = (rows[: pos + 1].double() @ q_att.double().T).T * scale          # [H, keys]
    return torch.softmax(s, dim=-1) @ rows[: pos + 1, :C].double()       # [H, C]


@pytest.mark.parametrize("dtype,C,R,H", [(torch.float32, 24, 8, 3), (torch.bfloat16, 32, 16, 4), (torch.bfloat16, 40, 12, 2),
                                         (torch.float32, 300, 20, 2), (torch.bfloat16, 256, 64, 20), (torch.bfloat16, 96, 32, 16)])
def test_attention_over_cached_latents_finds_one_key_among_hundreds(dtype, C, R, H):
    """420 cached rows over pages of 8 in shuffled order; for each probed key position (the first token, both sides of page
    borders, far back, the query's own) the query is made to point at that key, so the output must be that row's latent --
    a kernel that skips, repeats or misplaces one key of a page shows at once.  Single tokens and short portions (in bf16 with
    suitable sizes: the kernel whose tile rows are the heads), and prompt-sized portions."""
    ops = _ops()
    g = torch.Generator().manual_seed(8)
    bs, n, scale = 8, 420, 0.3
    pages = torch.randperm(70, generator=g)[:53].add(1).tolist()
    rows = torch.randn(n, C + R, generator=g).to(dtype)
    probes = [0, 1, 7, 8, 9, 199, 200, 391, 392, 418, 419]
    for j in probes:                                             # distinct long keys: a query along one of them sees mostly it
        rows[j] = rows[j] * 4
    pool = torch.zeros(72, 1, bs, C + R, dtype=dtype, device=DEV)
    for p in range(n):
        pool[pages[p // bs], 0, p % bs] = rows[p].to(DEV)
    bt = torch.zeros(3, 64, dtype=torch.int32, device=DEV)
    bt[2, :len(pages)] = torch.tensor(pages, dtype=torch.int32, device=DEV)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for T in (1, 5, 40):                                         # a decoded token; a short portion; a portion on the prompt kernel (bf16)
        pos0 = n - T
        q = torch.randn(T, H, C + R, generator=g) * 0.1
        for i in range(T):
            for h in range(H):
                j = probes[(i * H + h) % len(probes)]
                if j <= pos0 + i:
                    q[i, h] = rows[j].float() * (3.0 / scale / rows[j].float().pow(2).sum().sqrt())
        meta = _meta([(2, pos0, T)], {2: pages}, bs)
        out = ops.swa_sink_attn(q.view(T, -1).to(DEV).contiguous(), H, pool, None, bt, meta, None, scale, 1 << 30, latent_values=C)
        want = torch.stack([_attend_latents(q[i], rows.float(), scale, C, pos0 + i) for i in range(T)])
        _close(out.view(T, H, C), want, tol)


def test_batched_per_head_linear_with_sigmoid_gate():
    ops = _ops()
    g = torch.Generator().manual_seed(9)
    for dtype, K, N, tol in ((torch.float32, 10, 7, 1e-5), (torch.bfloat16, 16, 24, 2e-2), (torch.bfloat16, 12, 5, 2e-2)):
        T, B = 37, 3
        a = torch.randn(T, B * K + 4, generator=g).to(dtype)     # rows wider than the batches
        w = (torch.randn(B, N, K, generator=g) * K ** -0.5).to(dtype)
        gate = torch.randn(T, B + 2, generator=g)
        want = torch.einsum("tbk,bnk->tbn", a[:, :B * K].double().view(T, B, K), w.double())
        out = torch.full((T, B * (N + 3)), 7.0, device=DEV)      # fp32, batches N + 3 apart: the gaps stay untouched
        ops.batched_linear(a.to(DEV), w.to(DEV), out, a_batch_stride=K, out_batch_stride=N + 3)
        _close(out.view(T, B, N + 3)[..., :N], want, tol)
        assert (out.view(T, B, N + 3)[..., N:] == 7.0).all()
        typed = torch.zeros((T, B * N), dtype=dtype, device=DEV)
        ops.batched_linear(a.to(DEV), w.to(DEV), typed, a_batch_stride=K, out_batch_stride=N, gate=gate.to(DEV)[:, 2:])
        _close(typed.view(T, B, N), want * torch.sigmoid(gate[:, 2:].double())[:, :, None], max(tol, 1e-2 if dtype == torch.bfloat16 else 0))
