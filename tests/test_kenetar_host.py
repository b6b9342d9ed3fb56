"""CPU: host side of the post-norm hybrid decoder (Kenetar) -- configuration reader and its refusals, tensor names and
shapes, registry, rotary tables -- and properties of the plain restatement that the GPU tests lean on."""
import json
import math

import pytest
import torch

from vllm_neuron_b200.hybrid import DenseSpec, HybridConfig, RotSpec, random_weights, tensor_shapes


def _cfg(layers=None, bigram=True):
    moe = {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 6}}
    att = {"type": "latent_attention", "mlp": moe,
           "mixer": {"heads": 2, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 8, "q_rank": 10, "scale": 0.3,
                     "rot": {"dims": 4, "base": 100.0, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}}}}
    dl = {"type": "delta", "mlp": {"kind": "dense", "ff": 14}, "mixer": {"heads": 4, "kv_heads": 2, "dim": 3, "vdim": 5, "conv": 3}}
    emb = {"scale": 2.0}
    if bigram:
        emb["bigram"] = {"buckets": 11, "mul_prev": 3, "mul_cur": 5}
    return {"architecture": "Kenetar", "vocab": 20, "width": 12, "norm": {"eps": 1e-5}, "embedding": emb, "logit_scale": 2.5,
            "layers": layers if layers is not None else [dl, att, {**dl, "mlp": None}]}


def test_config_reader_round_trip_and_shapes():
    d = _cfg()
    cfg = HybridConfig.from_dict(d)
    assert cfg.style == "rms_post" and cfg.logit_scale == 2.5 and cfg.bigram == {"buckets": 11, "mul_prev": 3, "mul_cur": 5}
    assert cfg.to_dict() == d and HybridConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    m = cfg.layers[0].mixer
    assert (m.channels, m.proj) == (2 * 2 * 3 + 4 * 5, 32 + 8 + 20) and isinstance(cfg.layers[0].mlp, DenseSpec)
    assert cfg.layers[1].mlp.route == "softmax_out" and cfg.layers[2].mlp is None
    sh = tensor_shapes(cfg)
    assert sh["bigram"] == (12, 12) and sh["final.norm"] == (12,) and "final.norm.alpha" not in sh and "l0.norm1b" not in sh
    assert sh["l0.mix.q"] == (6, 12) and sh["l0.mix.k.conv"] == (6, 3) and sh["l0.mix.v.conv"] == (20, 3) and sh["l0.mix.b"] == (4, 12)
    assert sh["l0.mix.norm"] == (5,) and sh["l0.mix.g"] == (20, 12) and sh["l0.mix.o"] == (12, 20) and sh["l0.mlp.gate"] == (14, 12)
    assert sh["l1.mix.uq"] == (2 * 10, 10) and sh["l1.mix.dkv"] == (12, 12) and sh["l1.mix.dkv.norm"] == (8,)
    assert sh["l1.mix.uk"] == (12, 8) and sh["l1.mix.uv"] == (10, 8) and sh["l1.mix.g"] == (2, 12) and sh["l1.mix.o"] == (12, 10)
    assert sh["l1.mlp.router.b"] == (3,) and sh["l1.mlp.e2.down"] == (12, 6) and "l2.norm2" not in sh
    assert set(random_weights(cfg)) == set(sh)
    assert "bigram" not in tensor_shapes(HybridConfig.from_dict(_cfg(bigram=False)))
    bad_rot = json.loads(json.dumps(d["layers"][1]))
    bad_rot["mixer"]["rot"]["dims"] = 6
    for bad in ({"type": "mamba2", "mlp": None, "mixer": {"heads": 2, "vdim": 3, "state": 5, "groups": 1, "conv": 3}},
                {"type": "delta", "mlp": None, "mixer": {"heads": 3, "kv_heads": 2, "dim": 4, "vdim": 4, "conv": 2}}, bad_rot,
                {**d["layers"][0], "mlp": {"kind": "conv"}}):
        with pytest.raises(ValueError):
            HybridConfig.from_dict(_cfg(layers=[bad]))


def test_registry_picks_the_model_class_by_config():
    from vllm_neuron_b200 import registry

    arch, entry = registry.resolve(_cfg())
    assert arch == "Kenetar" and entry.family == "hybrid" and torch.float32 in entry.dtypes and torch.bfloat16 in entry.dtypes
    assert isinstance(entry.read_config(_cfg()), HybridConfig)


def test_rotary_tables_follow_the_blend_of_plain_and_stretched_frequencies():
    from oracle.kenetar_ref import yarn_angles

    for dims, base, sc in ((8, 100.0, {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}), (6, 10000.0, None),
                           (32, 20000.0, {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0})):
        cos, sin = RotSpec(dims, base, sc).tables(200)
        rc, rs = yarn_angles({"dims": dims, "base": base, "scaling": sc}, range(200), torch.float64)
        assert cos.shape == (200, dims // 2) and (cos.double() - rc).abs().max() < 1e-6 and (sin.double() - rs).abs().max() < 1e-6
    # by hand, dims 8 / base 100 / original 16: dim(t) = 8 ln(16 / (2 pi t)) / (2 ln 100); fast 4 -> -0.39, slow 1 -> 0.81:
    # lo = 0, hi = 1, so pair 0 keeps its frequency and every other pair is divided by the factor
    cos, sin = RotSpec(8, 100.0, {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}).tables(3)
    ms = 0.1 * math.log(4.0) + 1
    f = [1.0, 100 ** -0.25 / 4, 100 ** -0.5 / 4, 100 ** -0.75 / 4]
    for i, fi in enumerate(f):
        assert abs(cos[2, i].item() - math.cos(2 * fi) * ms) < 1e-6 and abs(sin[2, i].item() - math.sin(2 * fi) * ms) < 1e-6


def test_restatement_is_causal_and_carries_the_previous_token():
    """A later token never changes an earlier logit; the second token's embedding depends on the first (bigram row)."""
    from oracle import kenetar_ref

    d = _cfg()
    W = random_weights(HybridConfig.from_dict(d), seed=3)
    toks = [3, 7, 7, 1, 19, 4, 0, 7]
    full = kenetar_ref.forward(d, W, toks)
    assert (kenetar_ref.forward(d, W, toks[:5]) - full[:5]).abs().max() < 1e-12
    Wd = {k: v.double() for k, v in W.items()}
    a = kenetar_ref.embed_tokens([3, 7], Wd, d["embedding"])
    b = kenetar_ref.embed_tokens([4, 7], Wd, d["embedding"])
    assert (a[1] - b[1]).abs().max() > 1e-3
    assert torch.equal(kenetar_ref.embed_tokens([7], Wd, d["embedding"])[0], Wd["embed"][7] * 2.0 + Wd["bigram"][11])
