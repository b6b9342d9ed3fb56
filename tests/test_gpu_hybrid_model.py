"""GPU: the hybrid decoder through the stand-alone engine (runner step, page pool, state slots) against the plain
restatement on whole sequences: whole prompts, token-by-token decoding, ragged portions down to two tokens, mixed batches
with rows and pages that are freed and reused, long decoding past the window, and greedy generation through the scheduler.
The 32-bit mode is held to 1e-4 of the logit spread; the bf16 mode to its rounding noise."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _layer(kind, mlp, **mixer):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def _moe(experts, top, ff, limit, shared=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit},
            "shared": {"ff": shared, "limit": limit * 1.5} if shared else None}


def cfg_a():
    """GQA, top 2 of 6, window 9 over pages of 32, a layer without feed-forward, one without shared expert, one attention
    layer outside the value mixing, no window on the last one; in-projection K = 24 and inner = 20 (not a multiple of 8)."""
    att = dict(heads=4, kv_heads=2, dim=24, vdim=16, scale=0.2)
    return {"architecture": "Pumopel", "vocab": 90, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.7}, "layers": [
        _layer("attention", _moe(6, 2, 20, 1.1, 24), mask={"size": 9}, v_mix=True, **att),
        _layer("mamba2", None, heads=4, vdim=5, state=12, groups=2, conv=3, norm_groups=1),
        _layer("attention", _moe(6, 2, 20, 1.1), mask={"size": 33}, v_mix=True, **att),
        _layer("mamba2", _moe(3, 3, 8, 2.0, 8), heads=2, vdim=16, state=40, groups=1, conv=5, norm_groups=4),
        _layer("attention", _moe(6, 1, 20, 1.1, 24), v_mix=False, heads=2, kv_heads=2, dim=8, vdim=32, scale=0.35),
    ]}


def cfg_b():
    """State-space first, groups == heads, two taps, top 1; every GEMM on the tensor-core path and head sizes (32 / 16) that
    put prompt portions of 16 tokens or more on the tensor-core attention kernel."""
    return {"architecture": "Pumopel", "vocab": 200, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5}, "layers": [
        _layer("mamba2", _moe(4, 1, 16, 1.5, 32), heads=4, vdim=8, state=8, groups=4, conv=2, norm_groups=2),
        _layer("attention", _moe(4, 1, 16, 1.5, 32), heads=4, kv_heads=2, dim=32, vdim=16, scale=0.18, mask={"size": 40}, v_mix=True),
        _layer("attention", None, heads=4, kv_heads=2, dim=32, vdim=16, scale=0.18, mask={"size": 5}, v_mix=True),
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
        self.tol = 1e-4 if dtype == "float32" else 0.06
        self._ref = {}

    def tokens(self, n, seed):
        return torch.randint(0, self.cfg.vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()

    def ref(self, toks):
        from oracle import pumopel_ref

        key = tuple(toks)
        if key not in self._ref:
            self._ref[key] = pumopel_ref.forward(self.cfgd, self.W, toks)
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

    def err(self, got, toks):
        return self.errs(got, toks).max().item()

    def check(self, got, reqs):
        """32-bit: every position inside the bar.  bf16: the router sees bf16-rounded activations, so among hundreds of
        routing decisions of random weights a few near-ties go to the other expert than in the fp64 restatement and that
        token (and, faintly, later ones) moves by a whole expert; hence a bar on the bulk and on the median, not the max."""
        e = torch.cat([self.errs(got[i], toks) for i, toks in reqs.items()])
        if self.dtype == "float32":
            assert e.max().item() < self.tol, e.max().item()
        else:
            assert (e > self.tol).float().mean().item() <= 0.1 and e.median().item() < self.tol / 2, (e.max().item(), e.median().item())


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
    sizes = _portions(150, [2, 3, 2, 27, 30, 2, 1, 33, 7, 31, 1, 1, 10])     # cuts inside pages, windows and at their edges
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
    """A configuration drawn at random: 2-6 layers in any order, head counts / sizes / windows / taps / expert counts that
    need not be multiples of anything, some layers without feed-forward, window or value mixing."""
    heads = rng.choice([2, 4, 6, 8])
    kv = rng.choice([h for h in (1, 2, 3, 4, 6, 8) if heads % h == 0])
    dim, vdim = rng.choice([16, 24, 40, 64, 96, 128]), rng.choice([16, 24, 32, 48, 80, 136])
    sh = rng.choice([2, 4, 6, 12])
    sg = rng.choice([g for g in (1, 2, 3, 4, 6) if sh % g == 0])
    sv, sn = rng.choice([16, 33, 48, 64, 80]), rng.choice([16, 24, 48, 64, 96, 130])
    ng = rng.choice([g for g in (1, 2, 4, sh) if (sh * sv) % g == 0])
    conv = rng.choice([1, 2, 3, 4])
    experts, top = rng.choice([(4, 1), (4, 4), (8, 2), (16, 1), (32, 4)])
    ff, lim, shared = rng.choice([16, 40, 64]), rng.choice([1.0, 1.5, 7.0]), rng.choice([0, 32, 72])
    layers = []
    for _ in range(rng.randint(2, 6)):
        mlp = None if rng.random() < 0.15 else _moe(experts, top, ff, lim, shared or None)
        if rng.random() < 0.5:
            layers.append(_layer("mamba2", mlp, heads=sh, vdim=sv, state=sn, groups=sg, conv=conv, norm_groups=ng))
        else:
            m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=rng.choice([dim ** -0.5, 0.1, 0.3]), v_mix=rng.random() < 0.8)
            if rng.random() < 0.85:
                m["mask"] = {"size": rng.choice([1, 2, 17, 64, 100, 200])}
            layers.append(_layer("attention", mlp, **m))
    return {"architecture": "Pumopel", "vocab": rng.choice([100, 257, 512]), "width": rng.choice([64, 96, 136, 192, 256]),
            "norm": {"eps": rng.choice([1e-6, 1e-5])}, "embedding": {"scale": rng.choice([0.5, 1.0, 2.0])}, "layers": layers}


@pytest.mark.parametrize("seed", [2, 5, 12, 19, 22])
def test_random_configurations_in_32_bit(seed):
    """Whole prompt (long enough for the segmented scan and the wide expert tiles), ragged portions and a mixed batch of a
    prompt beside a decoding request, for configurations nobody picked by hand."""
    import random

    c = Case(_random_cfg(random.Random(seed)), "float32", seed=seed, max_num_seqs=3, pool_tokens=1024)
    toks, short = c.tokens(420, 50 + seed), c.tokens(30, 60 + seed)
    c.check(c.replay({"w": toks}, [[("w", 420)]]), {"w": toks})
    c.check(c.replay({"p": toks}, [[("p", n)] for n in _portions(420, [2, 3, 130, 1, 33, 7, 64, 1, 1, 257])]), {"p": toks})
    mixed = c.replay({"a": toks, "b": short}, [[("a", 300), ("b", 1)]] + [[("a", 1), ("b", 1)] for _ in range(29)] + [[("a", 91)]])
    c.check(mixed, {"a": toks, "b": short})


def test_long_decoding_past_every_window():
    c = Case(cfg_a(), "float32", max_num_seqs=2, pool_tokens=512)
    toks = c.tokens(300, 3)
    got = c.replay({"x": toks}, [[("x", 20)]] + [[("x", 1)] for _ in range(280)])
    c.check(got, {"x": toks})


def test_pool_exhaustion_is_refused():
    c = Case(cfg_b(), "bfloat16", max_num_seqs=2, pool_tokens=64)
    with pytest.raises(RuntimeError, match="KV pool exhausted"):
        c.replay({"x": c.tokens(100, 4)}, [[("x", 100)]])


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


def test_served_from_a_checkpoint_directory(tmp_path):
    """config.json + model.safetensors on disk -> registry -> engine; same logits as the in-memory weights."""
    import json

    from safetensors.torch import save_file
    from vllm_neuron_b200.engine import B200Engine

    c = Case(cfg_b(), "float32")
    with open(tmp_path / "config.json", "w") as f:
        json.dump(c.cfgd, f)
    save_file({k: v.contiguous() for k, v in c.W.items()}, str(tmp_path / "model.safetensors"))
    eng = B200Engine.from_pretrained(str(tmp_path), dtype="float32", max_num_seqs=2, max_pool_tokens=128)
    toks = c.tokens(50, 5)
    got = eng.replay_step([("r", toks, list(range(50)))], ["r"])["r"]
    assert c.err(got, toks) < 1e-4
