"""GPU: every mechanism of the hybrid decoder alone, against the plain restatement in oracle/pumopel_ref.py (fp64).
Sizes are deliberately awkward (odd widths, sizes that are not multiples of a warp or a page, top > 1, groups != heads)."""
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


def test_dyt_norm_and_fused_residual():
    ops = _ops()
    g = torch.Generator().manual_seed(0)
    T, W, top = 7, 50, 3
    x, y, y2 = (torch.randn(n, W, generator=g) * 2 for n in (T, T * top, T))
    w1, b1, w2, b2 = (torch.randn(W, generator=g) for _ in range(4))
    a1, a2 = 0.7, 1.3
    for odt, tol in ((torch.float32, 1e-6), (torch.bfloat16, 6e-3)):
        _close(ops.dyt_norm(x.to(DEV), w1.to(DEV), b1.to(DEV), a1, odt), torch.tanh(a1 * x.double()) * w1 + b1, tol)
        xd = x.to(DEV).clone()
        h = ops.dyt_residual(xd, y.to(DEV), (w1.to(DEV), b1.to(DEV), a1), (w2.to(DEV), b2.to(DEV), a2), odt, y2=y2.to(DEV), nsum=top)
        s = y.double().view(T, top, W).sum(1) + y2
        xr = x.double() + torch.tanh(a1 * s) * w1 + b1
        _close(xd, xr, 1e-6)                                  # the residual stream stays fp32 in both modes
        _close(h, torch.tanh(a2 * xr) * w2 + b2, tol)
    xd = x.to(DEV).clone()
    assert ops.dyt_residual(xd, y[:T].contiguous().to(DEV), (w1.to(DEV), b1.to(DEV), a1)) is None
    _close(xd, x.double() + torch.tanh(a1 * y[:T].double()) * w1 + b1, 1e-6)


@pytest.mark.parametrize("groups", [1, 3])
def test_gated_group_rmsnorm_gate_before_norm(groups):
    from oracle.pumopel_ref import rms_unit

    ops = _ops()
    g = torch.Generator().manual_seed(1)
    T, inner, eps = 5, 3 * 22, 1e-3
    y, w = torch.randn(T, inner, generator=g), torch.randn(inner, generator=g)
    zsrc = torch.randn(T, inner + 9, generator=g)            # z = the first `inner` columns of wider rows
    z = zsrc[:, :inner].double()
    want = rms_unit((y.double() * F.silu(z)).view(T, groups, -1), eps).reshape(T, inner) * w
    _close(ops.gated_group_rmsnorm(y.to(DEV), zsrc.to(DEV), w.to(DEV), groups, eps, torch.float32), want, 2e-6)
    wrong = rms_unit(y.double().view(T, groups, -1), eps).reshape(T, inner) * w * F.silu(z)   # gate after the norm
    assert (want - wrong).abs().max() > 0.05


def test_clamped_glu_limits():
    ops = _ops()
    g = torch.Generator().manual_seed(2)
    T, ff, limit = 6, 37, 1.25
    gu = torch.randn(T, 2 * ff, generator=g) * 3               # many values beyond +-limit
    gate, up = gu[:, :ff].double().clamp(max=limit), gu[:, ff:].double().clamp(-limit, limit)
    _close(ops.clamped_glu(gu.to(DEV), limit, torch.float32), gate * torch.sigmoid(1.702 * gate) * (up + 1), 2e-6)


@pytest.mark.parametrize("taps", [1, 2, 4, 5])
def test_causal_conv_ragged_portions_and_slot_reuse(taps):
    """Three sequences advance by portions of 1, 2 and more tokens per step; a slot is then handed to a NEW sequence while it
    still holds the old one's inputs.  Every step's output must equal the whole-sequence convolution."""
    from oracle.pumopel_ref import causal_conv_silu

    ops = _ops()
    g = torch.Generator().manual_seed(3)
    C, col0, ld = 45, 6, 60
    cw, cb = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    state = torch.full((4, max(taps - 1, 1), C), 7.0, device=DEV)  # garbage: a fresh sequence must not read it (one unused row when taps == 1)
    seqs = {s: torch.randn(n, ld, generator=g) for s, n in ((0, 11), (1, 4), (2, 9), (3, 6))}
    want = {s: causal_conv_silu(u[:, col0:col0 + C].double(), cw.double(), cb.double()) for s, u in seqs.items()}
    slot = {0: 2, 1: 0, 2: 3, 3: 0}                           # sequence 3 reuses sequence 1's slot
    plan = [[(0, 5), (1, 1), (2, 2)], [(0, 1), (1, 3), (2, 1)], [(0, 2), (2, 6), (3, 1)], [(0, 3), (3, 2)], [(3, 3)]]
    done = {s: 0 for s in seqs}
    for step in plan:
        entries = [(slot[s], done[s], n) for s, n in step]
        src = torch.cat([seqs[s][done[s]:done[s] + n] for s, n in step]).to(DEV)
        out = ops.causal_conv_silu(src, col0, C, cw.to(DEV), cb.to(DEV), state, _meta(entries, {slot[s]: [1] * 16 for s, _ in step}), torch.float32)
        o = 0
        for s, n in step:
            _close(out[o:o + n], want[s][done[s]:done[s] + n], 3e-6)
            o += n
            done[s] += n


SHORT_PLAN = ({0: 19, 1: 3, 2: 8}, [[(0, 7), (1, 1)], [(0, 1), (1, 2), (2, 2)], [(0, 11), (2, 6)]])
# portions of 256 tokens and more are cut into parallel segments of 128: ragged last segments (44, 1 and 15 tokens), a
# segmented portion that continues from a state left by an earlier segmented one, short sequences in the same step
LONG_PLAN = ({0: 700, 1: 3, 2: 300}, [[(0, 300), (1, 1)], [(0, 1), (1, 2), (2, 257)], [(0, 399), (2, 43)]])


@pytest.mark.parametrize("plan", [SHORT_PLAN, LONG_PLAN], ids=["short", "segmented"])
@pytest.mark.parametrize("H,G,P,N", [(4, 2, 5, 12), (3, 3, 40, 40), (2, 1, 33, 70), (2, 2, 100, 64), (1, 1, 70, 130)])
def test_selective_scan_ragged(H, G, P, N, plan):
    from oracle.pumopel_ref import selective_scan

    ops = _ops()
    g = torch.Generator().manual_seed(4)
    C = H * P + 2 * G * N
    a_log, dt_bias, d = torch.randn(H, generator=g) * 0.5, torch.randn(H, generator=g), torch.randn(H, generator=g)
    lens, plan = plan
    xbc = {s: torch.randn(n, C, generator=g) for s, n in lens.items()}
    dts = {s: torch.randn(n, H + 3, generator=g) * 2 for s, n in lens.items()}   # dt = columns 3.. of wider rows
    want = {}
    for s, n in lens.items():
        x = xbc[s][:, :H * P].double().view(n, H, P)
        B = xbc[s][:, H * P:H * P + G * N].double().view(n, G, N).repeat_interleave(H // G, 1)
        Cm = xbc[s][:, H * P + G * N:].double().view(n, G, N).repeat_interleave(H // G, 1)
        want[s] = selective_scan(x, B, Cm, dts[s][:, 3:].double(), dt_bias.double(), a_log.double(), d.double()).reshape(n, H * P)
    state = torch.full((3, H, P, N), 5.0, device=DEV)
    done = {s: 0 for s in lens}
    for step in plan:
        entries = [(s, done[s], n) for s, n in step]
        xs = torch.cat([xbc[s][done[s]:done[s] + n] for s, n in step]).to(DEV)
        ds = torch.cat([dts[s][done[s]:done[s] + n] for s, n in step]).to(DEV)
        meta = _meta(entries, {s: [1] * 128 for s, _ in step})
        assert (meta.scan_segs is not None) == (max(n for _, n in step) >= 2 * ops.SCAN_SEGMENT)
        y = ops.ssd_scan(xs, ds, 3, a_log.to(DEV), dt_bias.to(DEV), d.to(DEV), state, meta, H, P, N, G)
        o = 0
        for s, n in step:
            _close(y[o:o + n], want[s][done[s]:done[s] + n], 2e-5)
            o += n
            done[s] += n


def _attn_case(T, H, G, D, Dv, window, bs, *, spike=None, sink_val=None, seed=5):
    """Random q/k/v of one sequence; `spike` = (i, j, head): key j gets a score that dominates query i of that head."""
    g = torch.Generator().manual_seed(seed)
    q, k, v = torch.randn(T, H, D, generator=g), torch.randn(T, G, D, generator=g), torch.randn(T, G, Dv, generator=g)
    sink = torch.randn(H, generator=g) if sink_val is None else torch.full((H,), float(sink_val))
    if spike:
        i, j, h = spike
        k[j, h // (H // G)] = q[i, h] * 40.0 / q[i, h].norm() ** 2 * math.sqrt(D)   # score = 40 at scale 1/sqrt(D)
    return q, k, v, sink


def _run_attn(q, k, v, sink, window, bs, chunks, dtype=torch.float32):
    ops = _ops()
    T, H, D = q.shape
    G, Dv = k.shape[1], v.shape[2]
    nb = -(-T // bs)
    blocks = list(range(nb + 3, 3, -1))                        # descending, non-contiguous with the table order
    kp = torch.zeros(nb + 5, G, bs, D, dtype=dtype, device=DEV)
    vp = torch.zeros(nb + 5, G, bs, Dv, dtype=dtype, device=DEV)
    bt = torch.zeros(3, nb, dtype=torch.int32, device=DEV)
    bt[1, :nb] = torch.tensor(blocks, dtype=torch.int32)
    qkv = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1).to(DEV)
    outs, pos = [], 0
    for n in chunks:
        m = _meta([(1, pos, n)], {1: blocks}, bs)
        rows = qkv[pos:pos + n].contiguous()
        ops.kv_write_vmix(rows, H * D, H * D + G * D, kp, vp, m.slot_mapping)
        outs.append(ops.swa_sink_attn(rows, H, kp, vp, bt, m, sink.to(DEV), 1 / math.sqrt(D), window))
        pos += n
    return torch.cat(outs)


@pytest.mark.parametrize("chunks", [[70], [64, 1, 1, 1, 1, 1, 1], [2, 31, 30, 7]])
def test_attention_window_edges_sink_and_pages(chunks):
    """Window 17 over pages of 8 tokens: the last query's dominant key sits just INSIDE the window (it must take the output)
    or just OUTSIDE (it must not show at all); the same through decoded tokens and ragged portions."""
    from oracle.pumopel_ref import sink_window_attention

    T, H, G, D, Dv, window, bs = 70, 6, 2, 24, 40, 17, 8
    for j, inside in ((T - window, True), (T - 1 - window, False), (T - 1, True), (0, False)):
        q, k, v, sink = _attn_case(T, H, G, D, Dv, window, bs, spike=(T - 1, j, 4))
        want = sink_window_attention(q.double(), k.double(), v.double(), sink.double(), 1 / math.sqrt(D), window)
        got = _run_attn(q, k, v, sink, window, bs, chunks)
        _close(got, want, 2e-5)
        head = got[T - 1].view(H, Dv)[4].cpu()
        assert ((head - v[j, 4 // (H // G)]).abs().max() < 1e-3) == inside
    # a sink that dominates every score empties the output; a sink far below changes nothing
    q, k, v, sink = _attn_case(T, H, G, D, Dv, window, bs, sink_val=60.0)
    assert _run_attn(q, k, v, sink, window, bs, chunks).abs().max() < 1e-6
    q, k, v, sink = _attn_case(T, H, G, D, Dv, window, bs, sink_val=-60.0)
    want = sink_window_attention(q.double(), k.double(), v.double(), sink.double(), 1 / math.sqrt(D), window)
    _close(_run_attn(q, k, v, sink, window, bs, chunks), want, 2e-5)
    # bf16 pools: same mask, looser numbers
    q, k, v, sink = _attn_case(T, H, G, D, Dv, window, bs)
    want = sink_window_attention(q.double(), k.double(), v.double(), sink.double(), 1 / math.sqrt(D), window)
    _close(_run_attn(q, k, v, sink, window, bs, chunks, torch.bfloat16), want, 3e-2)


@pytest.mark.parametrize("H,G,D,Dv", [(8, 2, 24, 40), (4, 2, 32, 16), (6, 2, 20, 70), (16, 4, 64, 136)])
def test_warp_attention_shares_key_rows_between_query_heads(H, G, D, Dv):
    """Steps with many tokens on the CUDA-core kernel (fp32 pools; bf16 pools with head sizes the tensor-core kernel does not
    take): one CTA serves 4 or 2 query heads of a kv head (8/2, 16/4 and 4/2 heads), or 1 (6/2).  A dominant key just inside
    and just outside the window of the last query, per head."""
    from oracle.pumopel_ref import sink_window_attention

    T, window, bs = 420, 50, 8
    for head in (0, H - 1):
        for j, inside in ((T - window, True), (T - 1 - window, False)):
            q, k, v, sink = _attn_case(T, H, G, D, Dv, window, bs, spike=(T - 1, j, head))
            want = sink_window_attention(q.double(), k.double(), v.double(), sink.double(), 1 / math.sqrt(D), window)
            got = _run_attn(q, k, v, sink, window, bs, [400, 20])
            _close(got, want, 2e-5)
            row = got[T - 1].view(H, Dv)[head].cpu()
            assert ((row - v[j, head // (H // G)]).abs().max() < 1e-3) == inside
    if D % 16 or Dv % 16:
        q, k, v, sink = _attn_case(T, H, G, D, Dv, window, bs)
        want = sink_window_attention(q.double(), k.double(), v.double(), sink.double(), 1 / math.sqrt(D), window)
        _close(_run_attn(q, k, v, sink, window, bs, [T], torch.bfloat16), want, 3e-2)


@pytest.mark.parametrize("chunks", [[150], [16, 64, 3, 67], [33, 1, 1, 17, 98]])
def test_tensor_core_prompt_attention_edges(chunks):
    """bf16 pools, head sizes 32 / 48: portions of 16 tokens or more run on the mma.sync kernel (64-row tiles, 32-key tiles
    over pages of 8), shorter ones on the CUDA-core kernel.  A dominant key just inside / outside the window of a query in
    the middle of a tile and of the last query, against the restatement on the bf16-rounded q / k / v."""
    from oracle.pumopel_ref import sink_window_attention

    T, H, G, D, Dv, window, bs = 150, 4, 2, 32, 48, 37, 8
    for i in (T - 1, 100, 40):
        for j, inside in ((i - window + 1, True), (i - window, False), (i, True)):
            q, k, v, sink = _attn_case(T, H, G, D, Dv, window, bs, spike=(i, j, 3), seed=11)
            qb, kb, vb = (x.bfloat16().float() for x in (q, k, v))
            want = sink_window_attention(qb.double(), kb.double(), vb.double(), sink.double(), 1 / math.sqrt(D), window)
            got = _run_attn(qb, kb, vb, sink, window, bs, chunks, torch.bfloat16)
            _close(got, want, 1.5e-2)
            head = got[i].float().view(H, Dv)[3].cpu()
            assert ((head - vb[j, 3 // (H // G)]).abs().max() < 3e-2) == inside, (i, j)


def test_far_key_among_hundreds_without_window():
    """No window: key 3 of 400 must still decide the last query (pages of 32)."""
    from oracle.pumopel_ref import sink_window_attention

    T, H, G, D, Dv = 400, 2, 2, 16, 8
    q, k, v, sink = _attn_case(T, H, G, D, Dv, 1 << 30, 32, spike=(T - 1, 3, 1))
    got = _run_attn(q, k, v, sink, 1 << 30, 32, [T - 5, 1, 1, 1, 1, 1])
    _close(got, sink_window_attention(q.double(), k.double(), v.double(), sink.double(), 0.25, T + 1), 2e-5)
    assert (got[T - 1].view(H, Dv)[1].cpu() - v[3, 1]).abs().max() < 1e-3


def test_value_mixing_is_what_gets_cached():
    ops = _ops()
    g = torch.Generator().manual_seed(6)
    T, G, D, Dv, bs, lam = 5, 2, 4, 6, 4, 0.3
    rows = torch.randn(T, 3 + G * D + G * Dv, generator=g).to(DEV)
    rows2 = torch.randn(T, 3 + G * D + G * Dv, generator=g).to(DEV)
    m = _meta([(0, 0, T)], {0: [2, 1]}, bs)
    kp, vp = torch.zeros(3, G, bs, D, device=DEV), torch.zeros(3, G, bs, Dv, device=DEV)
    vf = torch.zeros(T, G * Dv, device=DEV)
    ops.kv_write_vmix(rows, 3, 3 + G * D, kp, vp, m.slot_mapping, v_first=vf, mode=1)
    v1 = rows[:, 3 + G * D:]
    assert torch.equal(vf, v1)
    ops.kv_write_vmix(rows2, 3, 3 + G * D, kp, vp, m.slot_mapping, v_first=vf, lam=lam, mode=2)
    want = ((1 - lam) * rows2[:, 3 + G * D:] + lam * v1).view(T, G, Dv)
    got = torch.stack([vp[[2, 1][t // bs], :, t % bs] for t in range(T)])
    _close(got, want, 1e-6)
    _close(torch.stack([kp[[2, 1][t // bs], :, t % bs] for t in range(T)]), rows2[:, 3:3 + G * D].view(T, G, D), 1e-7)


@pytest.mark.parametrize("E,top,shared", [(5, 2, 0), (16, 1, 24), (7, 3, 10)])
def test_moe_weight_on_the_input(E, top, shared):
    """Router + experts + shared expert against the restatement; the routing weight must scale the expert's INPUT (the
    clamps make that differ from scaling its output)."""
    from oracle.pumopel_ref import moe_ff
    from vllm_neuron_b200.hybrid import HybridConfig, HybridCausalLM, random_weights

    W, ff, limit, T = 40, 12, 0.8, 45
    cfgd = {"architecture": "Pumopel", "vocab": 16, "width": W, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "layers": [{"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.3, "mask": {"size": 4}},
                        "mlp": {"kind": "moe", "router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": limit},
                                "shared": {"ff": shared, "limit": 2 * limit} if shared else None}}]}
    cfg = HybridConfig.from_dict(cfgd)
    Wt = random_weights(cfg, seed=7, std=0.4)
    model = HybridCausalLM(cfg, Wt, num_blocks=4, max_num_seqs=1, max_model_len=64, device=DEV, dtype=torch.float32)
    h = torch.randn(T, W, generator=torch.Generator().manual_seed(8))
    pairs, sh = model._moe(model.layers[0], h.to(DEV))
    got = pairs.view(T, top, W).sum(1) + (sh if sh is not None else 0)
    W64 = {k: v.double() for k, v in Wt.items()}
    want = moe_ff(h.double(), W64, "l0.mlp.", cfgd["layers"][0]["mlp"])
    _close(got, want, 2e-5)
    idx, wt = _ops().moe_topk(model._linear(h.to(DEV), model.layers[0]["w_router"]), top)
    ties = torch.tensor([[1.0, 3.0, 3.0, -2.0, 3.0]], device=DEV)            # equal logits: the lower index first
    assert _ops().moe_topk(ties, 2)[0].tolist() == [[1, 2]]
    s = torch.sigmoid(h.double() @ W64["l0.mlp.router"].T)
    val, ref_idx = s.topk(top, dim=-1)
    assert torch.equal(idx.cpu().long(), ref_idx) and (wt.cpu().double() - val).abs().max() < 1e-6


def test_moe_wide_tiles_match_the_default_tiles():
    """Prompt-sized bf16 batch: experts with 128-row tiles (ragged tails, an expert that gets almost nothing) give the same
    pairs as the 32-row tiles, and both follow the restatement evaluated on the bf16-rounded operands."""
    from oracle.pumopel_ref import clamped_glu_expert

    ops = _ops()
    E, top, W, ff, T, limit = 5, 2, 64, 24, 700, 0.9
    g = torch.Generator().manual_seed(21)
    h = torch.randn(T, W, generator=g).bfloat16()
    w_gu = (0.3 * torch.randn(E, 2 * ff, W, generator=g)).bfloat16()
    w_dn = (0.3 * torch.randn(E, W, ff, generator=g)).bfloat16()
    logits = torch.randn(T, E, generator=g)
    logits[:, 3] -= 6.0                                     # expert 3 is chosen a handful of times at most
    idx, wt = ops.moe_topk(logits.to(DEV), top)
    hd, gud, dnd = h.to(DEV), w_gu.to(DEV), w_dn.to(DEV)
    assert ops.moe_wide_tiles(hd, gud, T * top) == 4 * ops.moe_tile_rows()
    assert ops.moe_wide_tiles(hd, gud, 10) is None and ops.moe_wide_tiles(hd.float(), gud.float(), T * top) is None
    wide = ops.moe_experts(hd, wt, ops.moe_align(idx, E, 4 * ops.moe_tile_rows()), gud, dnd, top, limit)
    base = ops.moe_experts(hd, wt, ops.moe_align(idx, E), gud, dnd, top, limit)
    assert torch.equal(wide, base)                          # same K order per row: the tile height changes nothing
    want = torch.zeros(T * top, W, dtype=torch.float64)
    for pair in range(T * top):
        e = int(idx.view(-1)[pair])
        x = (h[pair // top].float() * wt.view(-1)[pair].cpu()).bfloat16().double()   # the weight goes into the operand
        Wd = {"gate": w_gu[e, :ff].double(), "up": w_gu[e, ff:].double(), "down": w_dn[e].double()}
        want[pair] = clamped_glu_expert(x[None], Wd, "", limit)[0]
    _close(wide, want, 1e-2)                                # the activation between the two GEMMs is rounded to bf16


def test_linear_paths_agree_with_matmul():
    ops = _ops()
    g = torch.Generator().manual_seed(9)
    for m, n, k in ((45, 70, 20), (3, 774, 256), (300, 129, 288)):
        a, w = torch.randn(m, k, generator=g), torch.randn(n, k, generator=g)
        _close(ops.linear_simt(a.to(DEV), w.to(DEV)), a.double() @ w.double().T, 2e-6)
        ab, wb = a.bfloat16(), w.bfloat16()
        want = ab.double() @ wb.double().T
        _close(ops.linear_simt(ab.to(DEV), wb.to(DEV)), want, 2e-5)   # K % 8 == 0: tensor cores, fp32 accumulation
        if k % 8 == 0:
            _close(ops.gemm(ab.to(DEV), wb.to(DEV), out_dtype=torch.float32), want, 2e-5)
