"""GPU: the post-norm hybrid decoder (Kenetar) through the stand-alone engine (runner step, page pool, state slots) against
the plain restatement on whole sequences: whole prompts, token-by-token decoding from the first token, ragged portions down
to two tokens, mixed batches with rows and pages that are freed and reused, long decoding, configurations drawn at random,
and greedy generation through the scheduler.  The 32-bit mode is held to 1e-4 of the logit spread; the bf16 mode to its
rounding noise."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _layer(kind, mlp, **mixer):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def _moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0, scaling=None, dims=None):
    return dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale,
                rot={"dims": dims or rot_dim, "base": base, "scaling": scaling})


def cfg_a():
    """Attention first, head counts that differ between the mixers, key heads == heads and a single key head, top 3 of 5 and
    top 1, two and five taps, a layer without feed-forward, widths (44, 20, 28) that keep GEMMs off the tensor cores in places,
    YaRN on one attention layer and plain angles on the other."""
    yarn = {"factor": 6.0, "original": 48, "fast": 12.0, "slow": 2.0}
    return {"architecture": "Kenetar", "vocab": 90, "width": 44, "norm": {"eps": 1e-5}, "logit_scale": 0.7,
            "embedding": {"scale": 3.0, "bigram": {"buckets": 37, "mul_prev": 5, "mul_cur": 11}}, "layers": [
        _layer("latent_attention", _moe(5, 3, 20), **_latent(3, 20, 12, 28, 24, 36, 0.21, 700.0, yarn)),
        _layer("delta", None, heads=4, kv_heads=4, dim=12, vdim=10, conv=2),
        _layer("delta", _dense(52), heads=2, kv_heads=1, dim=40, vdim=24, conv=5),
        _layer("latent_attention", _moe(3, 1, 16), **_latent(2, 8, 6, 16, 40, 20, 0.4, 50.0)),
        _layer("delta", _moe(5, 3, 20), heads=4, kv_heads=2, dim=12, vdim=10, conv=3),
    ]}


def cfg_b():
    """Delta first, no bigram table, every GEMM on the tensor-core path, and attention sizes (48 / 32 per cached row) that put
    prompt portions of 16 tokens or more on the tensor-core attention kernel; one tap."""
    yarn = {"factor": 2.0, "original": 32, "fast": 8.0, "slow": 1.0}
    return {"architecture": "Kenetar", "vocab": 200, "width": 64, "norm": {"eps": 1e-6}, "logit_scale": 1.5,
            "embedding": {"scale": 8.0}, "layers": [
        _layer("delta", _dense(96), heads=4, kv_heads=2, dim=16, vdim=32, conv=1),
        _layer("latent_attention", _moe(4, 2, 32), **_latent(4, 16, 16, 24, 32, 48, 0.17, 1000.0, yarn)),
        _layer("latent_attention", None, **_latent(4, 16, 16, 24, 32, 48, 0.17, 1000.0, yarn)),
        _layer("delta", _moe(4, 2, 32), heads=2, kv_heads=2, dim=64, vdim=16, conv=4),
    ]}


class Case:
    def __init__(self, cfgd, dtype, seed=0, max_num_seqs=3, pool_tokens=1024):
        from vllm_neuron_b200.engine import B200Engine
        from vllm_neuron_b200.hybrid import HybridConfig, random_weights

        self.cfgd, self.dtype = cfgd, dtype
        self.cfg = HybridConfig.from_dict(cfgd)
        self.W = random_weights(self.cfg, seed=seed)
        self.engine = B200Engine(self.cfg, self.W, dtype=dtype, max_num_seqs=max_num_seqs, max_pool_tokens=pool_tokens,
                                 max_num_batched_tokens=1 << 20)
        # bf16: every branch is renormalised to unit RMS before it joins the residual stream, so the rounding noise of a narrow
        # layer is not damped by a small branch; the restatement's distance to the bf16 engine is a few percent of the spread
        self.tol = 1e-4 if dtype == "float32" else 0.1
        self._ref = {}

    def tokens(self, n, seed):
        return torch.randint(0, self.cfg.vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()

    def ref(self, toks):
        from oracle import kenetar_ref

        key = tuple(toks)
        if key not in self._ref:
            self._ref[key] = kenetar_ref.forward(self.cfgd, self.W, toks)
        return self._ref[key]

    def replay(self, reqs, schedule):
        """reqs: id -> tokens; schedule: list of steps, each [(id, n)].  Logits of every position, per request."""
        at = {i: 0 for i in reqs}
        got = {i: [] for i in reqs}
        for step in schedule:
            entries, end = [], []
            for i, n in step:
                entries.append((i, reqs[i][at[i]:at[i] + n], list(range(n))))
                at[i] += n
                if at[i] == len(reqs[i]):
                    end.append(i)
            taps = self.engine.replay_step(entries, end)
            for i, n in step:
                assert taps[i].shape == (n, self.cfg.vocab)
                got[i].append(taps[i])
        assert all(at[i] == len(reqs[i]) for i in reqs)
        return {i: torch.cat(v) for i, v in got.items()}

    def errs(self, got, toks):
        want = self.ref(toks)
        d = got.double() - want
        d = d - d.mean(-1, keepdim=True)
        spread = (want - want.mean(-1, keepdim=True)).pow(2).mean().sqrt()
        return d.pow(2).mean(-1).sqrt() / spread

    def check(self, got, reqs):
        """32-bit: every position inside the bar.  bf16: the router sees bf16-rounded activations, so a few near-ties among
        hundreds of routing decisions go to another expert than in the fp64 restatement and move that token by a whole
        expert -- and, through the recurrent state, the tokens after it until the decay has worn the difference off; hence a
        bar on the bulk (three quarters of the positions) and on the median, not on the maximum.  A wrong kernel puts every
        position near 1."""
        e = torch.cat([self.errs(got[i], toks) for i, toks in reqs.items()])
        if self.dtype == "float32":
            assert e.max().item() < self.tol, e.max().item()
        else:
            assert e.quantile(0.75).item() < self.tol and e.median().item() < self.tol / 2, (e.max().item(), e.median().item())


def _portions(n, sizes):
    out, k = [], 0
    while n > 0:
        c = min(sizes[k % len(sizes)], n)
        out.append(c)
        n -= c
        k += 1
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg", [cfg_a, cfg_b])
def test_whole_prompt_decode_and_portions_agree_with_the_restatement(cfg, dtype):
    c = Case(cfg(), dtype)
    toks = c.tokens(150, 1)
    whole = c.replay({"w": toks}, [[("w", 150)]])
    c.check(whole, {"w": toks})
    short = c.tokens(45, 2)
    one_by_one = c.replay({"d": short}, [[("d", 1)] for _ in short])          # the first tokens, then decoding throughout
    c.check(one_by_one, {"d": short})
    sizes = _portions(150, [2, 3, 2, 27, 30, 2, 1, 33, 7, 31, 1, 1, 10])     # cuts inside pages and staging chunks, and at their edges
    cut = c.replay({"p": toks}, [[("p", n)] for n in sizes])
    c.check(cut, {"p": toks})
    d = (cut["p"] - whole["w"]).abs().max().item() / whole["w"].abs().max().item()
    assert d < (1e-5 if dtype == "float32" else 0.05), d                      # how the prompt was cut does not matter


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_with_reused_rows_and_pages(dtype):
    """Seven requests of unequal length (1 .. 130 tokens) through THREE rows and a pool that cannot hold them all at once:
    portions beside single tokens, requests that sit out steps, rows and pages taken over by later requests."""
    c = Case(cfg_a(), dtype, max_num_seqs=3, pool_tokens=320)
    lens = {"a": 130, "b": 1, "c": 37, "d": 2, "e": 64, "f": 33, "g": 90}
    reqs = {i: c.tokens(n, 10 + k) for k, (i, n) in enumerate(lens.items())}
    sched = [
        [("a", 40), ("b", 1), ("c", 2)],            # b ends: its row and page go back
        [("a", 1), ("c", 30), ("d", 1)],
        [("c", 1), ("d", 1)],                        # a sits out; d ends
        [("a", 25), ("c", 1), ("e", 31)],
        [("a", 1), ("c", 1), ("e", 1)],
        [("a", 1), ("c", 2), ("e", 32)],            # c and e end
        [("a", 62), ("f", 33), ("g", 2)],           # f is whole in one step and ends
        [("g", 60)],
        [("g", 1)], [("g", 1)],
        [("g", 26)],
    ]
    got = c.replay(reqs, sched)
    c.check(got, reqs)
    assert c.engine.pool.num_free == c.engine.num_blocks - 1 and not c.engine.scheduler.running
    if dtype == "float32":                                                     # each alone gives the same numbers
        alone = Case(cfg_a(), dtype, max_num_seqs=1, pool_tokens=160)
        for i in ("a", "e", "g"):
            solo = alone.replay({i: reqs[i]}, [[(i, len(reqs[i]))]])
            d = (solo[i] - got[i]).abs().max().item() / solo[i].abs().max().item()
            assert d < 1e-5, (i, d)


def _random_cfg(rng):
    """A configuration drawn at random: 2-6 layers in any order, head counts / sizes / ranks / taps / expert counts that
    need not be multiples of anything, dense, routed or no feed-forward, with or without bigram table and YaRN."""
    dh = rng.choice([2, 3, 4, 6])
    dg = rng.choice([g for g in (1, 2, 3, 4, 6) if dh % g == 0])
    dd, dv, conv = rng.choice([8, 24, 40, 64, 96, 260]), rng.choice([8, 20, 32, 72, 128]), rng.choice([1, 2, 3, 4, 7])
    ah = rng.choice([1, 2, 3, 4, 8])
    ad, ar, av = rng.choice([8, 16, 24, 40]), rng.choice([4, 8, 16, 32]), rng.choice([8, 16, 40, 80])
    rank, qrank = rng.choice([16, 24, 32, 80, 144]), rng.choice([16, 24, 72, 128])
    dims = ar if rng.random() < 0.7 else ar // 2
    scaling = None if rng.random() < 0.3 else {"factor": rng.choice([2.0, 4.0, 40.0]), "original": rng.choice([16, 64, 4096]),
                                              "fast": rng.choice([8.0, 32.0]), "slow": rng.choice([1.0, 2.0])}
    experts, top = rng.choice([(4, 1), (4, 4), (8, 2), (16, 1), (32, 4), (7, 3)])
    ff = rng.choice([16, 40, 64])
    layers = []
    for _ in range(rng.randint(2, 6)):
        r = rng.random()
        mlp = None if r < 0.15 else _dense(rng.choice([24, 64, 100])) if r < 0.4 else _moe(experts, top, ff)
        if rng.random() < 0.5:
            layers.append(_layer("delta", mlp, heads=dh, kv_heads=dg, dim=dd, vdim=dv, conv=conv))
        else:
            layers.append(_layer("latent_attention", mlp, **_latent(ah, ad, ar, av, rank, qrank, rng.choice([(ad + ar) ** -0.5, 0.1, 0.3]),
                                                                  rng.choice([100.0, 10000.0, 500000.0]), scaling, dims)))
    emb = {"scale": rng.choice([0.5, 1.0, 12.0])}
    if rng.random() < 0.8:
        emb["bigram"] = {"buckets": rng.choice([1, 17, 300]), "mul_prev": rng.choice([1, 31, 1000003]), "mul_cur": rng.choice([1, 7, 999983])}
    return {"architecture": "Kenetar", "vocab": rng.choice([100, 257, 512]), "width": rng.choice([64, 96, 136, 192, 256]),
            "norm": {"eps": rng.choice([1e-6, 1e-5])}, "logit_scale": rng.choice([0.25, 1.0, 3.0]), "embedding": emb, "layers": layers}


@pytest.mark.parametrize("seed", [1, 4, 7, 11, 13, 16])
def test_random_configurations_in_32_bit(seed):
    """Whole prompt (long enough for the wide expert tiles and many staging chunks), ragged portions and a mixed batch of a
    prompt beside a decoding request, for configurations nobody picked by hand."""
    import random

    c = Case(_random_cfg(random.Random(seed)), "float32", seed=seed, max_num_seqs=3, pool_tokens=1024)
    toks, short = c.tokens(420, 50 + seed), c.tokens(30, 60 + seed)
    c.check(c.replay({"w": toks}, [[("w", 420)]]), {"w": toks})
    c.check(c.replay({"p": toks}, [[("p", n)] for n in _portions(420, [2, 3, 130, 1, 33, 7, 64, 1, 1, 257])]), {"p": toks})
    mixed = c.replay({"a": toks, "b": short}, [[("a", 300), ("b", 1)]] + [[("a", 1), ("b", 1)] for _ in range(29)] + [[("a", 91)]])
    c.check(mixed, {"a": toks, "b": short})


@pytest.mark.parametrize("seed", [2, 9])
def test_random_configurations_in_bf16(seed):
    import random

    c = Case(_random_cfg(random.Random(seed)), "bfloat16", seed=seed, max_num_seqs=2, pool_tokens=512)
    toks = c.tokens(200, 70 + seed)
    c.check(c.replay({"p": toks}, [[("p", n)] for n in _portions(200, [40, 2, 1, 1, 65, 17])]), {"p": toks})


def test_long_decoding():
    c = Case(cfg_a(), "float32", max_num_seqs=2, pool_tokens=512)
    toks = c.tokens(300, 3)
    got = c.replay({"x": toks}, [[("x", 20)]] + [[("x", 1)] for _ in range(280)])
    c.check(got, {"x": toks})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(dtype):
    """engine.generate: five prompts over three rows, prompts cut by a 48-token budget next to decodes.  Every generated
    token must be the restatement's argmax given the same history (or lie within rounding noise of it)."""
    from vllm_neuron_b200.engine import B200Engine

    c = Case(cfg_b(), dtype)
    eng = B200Engine(c.cfg, c.W, dtype=dtype, max_num_seqs=3, max_pool_tokens=512, max_num_batched_tokens=48)
    prompts = [c.tokens(n, 20 + n) for n in (70, 3, 33, 1, 100)]
    outs = eng.generate(prompts, max_new_tokens=12)
    assert eng.pool.num_free == eng.num_blocks - 1
    exact = far = 0
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        ref = c.ref(p + o)
        for k, tok in enumerate(o):
            row = ref[len(p) + k - 1]
            best = int(row.argmax())
            exact += best == tok
            gap = (row[best] - row[tok]).item() / row.std().item()
            far += gap > (1e-4 if dtype == "float32" else 0.1)
    assert far <= (0 if dtype == "float32" else 3) and exact >= (60 if dtype == "float32" else 45), (far, exact)


def test_served_from_a_checkpoint_directory_and_layer_streams(tmp_path):
    """config.json + model.safetensors on disk -> registry -> engine; same logits as the in-memory weights, and the residual
    stream after every layer equals the restatement's."""
    import json

    from oracle import kenetar_ref
    from safetensors.torch import save_file
    from vllm_neuron_b200.engine import B200Engine
    from vllm_neuron_b200.registry import load_config

    c = Case(cfg_a(), "float32")
    with open(tmp_path / "config.json", "w") as f:
        json.dump(c.cfgd, f)
    save_file({k: v.contiguous() for k, v in c.W.items()}, str(tmp_path / "model.safetensors"))
    arch, entry, cfg = load_config(str(tmp_path))
    assert arch == "Kenetar" and entry.family == "hybrid" and cfg == c.cfg
    eng = B200Engine.from_pretrained(str(tmp_path), dtype="float32", max_num_seqs=2, max_pool_tokens=128)
    toks = c.tokens(50, 5)
    cap, fwd = [], eng.model.forward
    eng.model.forward = lambda tokens, meta, rows: fwd(tokens, meta, rows, capture=cap)
    got = eng.replay_step([("r", toks, list(range(50)))], ["r"])["r"]
    assert c.errs(got, toks).max().item() < 1e-4
    _, streams = kenetar_ref.forward(c.cfgd, c.W, toks, want_layers=True)
    assert len(cap) == len(c.cfgd["layers"])
    for got_x, want_x in zip(cap, streams):
        assert (got_x.double().cpu() - want_x).abs().max().item() < 1e-4 * want_x.abs().max().item()


def test_trace_replay_command_line(tmp_path):
    """bin/trace_run as a user runs it: a checkpoint folder, steps on standard input (two requests, portions beside single
    tokens, a step that reports nothing, a request that ends and frees its row), logits files per step."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np
    from safetensors.torch import save_file

    c = Case(cfg_b(), "float32")
    model_dir, out_dir = tmp_path / "model", tmp_path / "out"
    model_dir.mkdir()
    with open(model_dir / "config.json", "w") as f:
        json.dump(c.cfgd, f)
    save_file({k: v.contiguous() for k, v in c.W.items()}, str(model_dir / "model.safetensors"))
    a, b = c.tokens(70, 31), c.tokens(9, 32)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:33], "want": [0, 32]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[33:35], "want": []}, {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[8:], "want": [0]}, {"id": "a", "tokens": a[35:36], "want": [0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": a[36:], "want": [0, 33]}], "end": ["a"]},
    ]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(model_dir), "--dtype", "float32",
                        "--out", str(out_dir), "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [ln for ln in p.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb = c.ref(a), c.ref(b)
    want = {0: [ra[0], ra[32]], 1: [rb[7]], 2: [rb[8], ra[35]], 3: [ra[36], ra[69]]}
    for n, rows in want.items():
        got = np.fromfile(out_dir / f"{n}.f32", dtype="<f4").reshape(len(rows), -1)
        for g, w in zip(got, rows):
            d = torch.from_numpy(g).double() - w
            assert (d - d.mean()).pow(2).mean().sqrt().item() < 1e-4 * (w - w.mean()).pow(2).mean().sqrt().item()
