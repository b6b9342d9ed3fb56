"""CPU: host side of the hybrid decoder -- configuration reader, registry, ragged-step index construction, page pool and
engine scheduler -- and properties of the plain restatement that the GPU tests lean on."""
import json

import pytest
import torch

from vllm_neuron_b200.core.engine_scheduler import BlockPool, EngineRequest, EngineScheduler
from vllm_neuron_b200.hybrid import HybridConfig, StepMeta, random_weights, tensor_shapes


def _cfg(window=4, layers=None):
    moe = {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 6, "limit": 1.0}, "shared": {"ff": 4, "limit": 2.0}}
    att = {"type": "attention", "mlp": moe, "mixer": {"heads": 2, "kv_heads": 1, "dim": 6, "vdim": 4, "scale": 0.4,
                                                     "mask": {"size": window}, "v_mix": True}}
    ssm = {"type": "mamba2", "mlp": None, "mixer": {"heads": 2, "vdim": 3, "state": 5, "groups": 1, "conv": 3, "norm_groups": 2}}
    return {"architecture": "Pumopel", "vocab": 20, "width": 12, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
            "layers": layers if layers is not None else [att, ssm, att]}


def test_config_reader_round_trip_and_shapes():
    d = _cfg()
    cfg = HybridConfig.from_dict(d)
    assert cfg.to_dict() == d and HybridConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    m = cfg.layers[1].mixer
    assert (m.inner, m.channels, m.proj) == (6, 16, 24) and cfg.layers[1].mlp is None
    assert cfg.layers[0].mlp.top == 2 and cfg.layers[0].mlp.shared_ff == 4 and cfg.layers[0].mixer.window == 4
    sh = tensor_shapes(cfg)
    assert sh["l1.mix.in"] == (24, 12) and sh["l1.mix.conv"] == (16, 3) and sh["l0.mix.q"] == (12, 12) and sh["l0.mix.v"] == (4, 12)
    assert sh["l2.mlp.e2.down"] == (12, 6) and sh["l0.mlp.shared.gate"] == (4, 12) and sh["l0.mix.vmix"] == ()
    assert "l1.norm2" not in sh and "l1.mlp.router" not in sh
    assert set(random_weights(cfg)) == set(sh)
    for bad in ({"type": "lstm", "mixer": {}, "mlp": None},
                {"type": "attention", "mlp": None, "mixer": {"heads": 3, "kv_heads": 2, "dim": 4, "vdim": 4, "scale": 1.0}}):
        with pytest.raises(ValueError):
            HybridConfig.from_dict(_cfg(layers=[bad]))


def test_registry_picks_the_model_class_by_config():
    from vllm_neuron_b200 import registry

    arch, entry = registry.resolve(_cfg())
    assert arch == "Pumopel" and entry.family == "hybrid" and torch.float32 in entry.dtypes
    assert isinstance(entry.read_config(_cfg()), HybridConfig)
    arch, entry = registry.resolve({"architectures": ["Qwen2ForCausalLM"]})
    assert entry.family == "dense" and entry.dtypes == (torch.bfloat16,)
    with pytest.raises(ValueError, match="not served"):
        registry.resolve({"architectures": ["NoSuchModel"]})


def test_step_meta_positions_and_slots():
    m = StepMeta.build([(2, 0, 5), (0, 30, 4), (1, 7, 1)], {2: [9, 3], 0: [4, 6], 1: [8]}, 32, "cpu")
    assert m.num_seqs == 3 and m.num_tokens == 10
    assert m.seq_start.tolist() == [0, 5, 9, 10] and m.seq_slot.tolist() == [2, 0, 1] and m.seq_pos0.tolist() == [0, 30, 7]
    assert m.tok_seq.tolist() == [0] * 5 + [1] * 4 + [2] and m.tok_row.tolist() == [2] * 5 + [0] * 4 + [1]
    assert m.tok_pos.tolist() == [0, 1, 2, 3, 4, 30, 31, 32, 33, 7]
    assert m.slot_mapping.tolist() == [288, 289, 290, 291, 292, 4 * 32 + 30, 4 * 32 + 31, 6 * 32, 6 * 32 + 1, 8 * 32 + 7]
    assert m.slot_mapping.dtype == torch.int64 and m.tok_pos.dtype == torch.int32


def test_step_meta_cuts_long_portions_into_scan_segments():
    from vllm_neuron_b200 import ops
    from vllm_neuron_b200.hybrid import StepMeta

    seg = ops.SCAN_SEGMENT
    rows = {r: [1] * 64 for r in range(3)}
    short = StepMeta.build([(0, 0, 2 * seg - 1), (1, 5, 1)], rows, 32, "cpu")
    assert short.scan_segs is None and short.num_segs == 0
    m = StepMeta.build([(0, 0, 2 * seg + 44), (1, 5, 1), (2, 7, 2 * seg)], rows, 32, "cpu")
    a = 2 * seg + 44
    assert m.scan_segs.tolist() == [[0, seg, 0, 1], [seg, 2 * seg, 0, 0], [2 * seg, a, 0, 2], [a, a + 1, 1, 3],
                                    [a + 1, a + 1 + seg, 2, 1], [a + 1 + seg, a + 1 + 2 * seg, 2, 2]]
    assert m.scan_seq_seg0.tolist() == [0, 3, 4, 6] and m.num_segs == 6


def test_block_pool_reuses_freed_pages_and_never_hands_out_page_zero():
    p = BlockPool(6)
    a = p.allocate(3)
    assert a == [1, 2, 3] and p.num_free == 2
    p.free(a[:2])
    assert p.allocate(2) == [1, 2]
    with pytest.raises(RuntimeError, match="exhausted"):
        p.allocate(3)
    assert 0 not in p.allocate(2) and p.num_free == 0


def _req(i, n, new=4):
    return EngineRequest(i, list(range(n)), n, new)


def test_mixed_policy_shares_a_token_budget_between_decodes_and_prompt_portions():
    s = EngineScheduler(BlockPool(40), block_size=8, max_num_seqs=2, max_model_len=200, max_num_batched_tokens=20, policy="mixed")
    for r in (_req("a", 30), _req("b", 5), _req("c", 3)):
        s.add(r)
    o = s.schedule()
    assert o.num_scheduled_tokens == {"a": 20} and [n.req_id for n in o.scheduled_new_reqs] == ["a"]
    assert len(o.scheduled_new_reqs[0].block_ids[0]) == 3 and len(o.scheduled_new_reqs[0].prompt_token_ids) == 30
    s.update(o, {})
    o = s.schedule()                       # the rest of a's prompt, and b beside it; c waits for a free line
    assert o.num_scheduled_tokens == {"a": 10, "b": 5} and o.scheduled_cached_reqs.req_ids == ["a"]
    assert o.scheduled_cached_reqs.new_block_ids == [([4],)]
    s.update(o, {"a": [7], "b": [7]})
    o = s.schedule()
    assert o.num_scheduled_tokens == {"a": 1, "b": 1} and not o.scheduled_new_reqs
    a = s.running[0]
    done = []
    for _ in range(3):
        done += s.update(o, {"a": [1], "b": [1]})
        o = s.schedule()
    assert {r.req_id for r in done} == {"a", "b"} and a.finished == "length" and a.block_ids == []
    assert set(o.finished_req_ids) == {"a", "b"} and [n.req_id for n in o.scheduled_new_reqs] == ["c"]
    assert s.pool.num_free == 39 - 1


def test_exclusive_policy_prefills_alone():
    s = EngineScheduler(BlockPool(40), block_size=8, max_num_seqs=2, max_model_len=200, policy="exclusive")
    s.add(_req("a", 10))
    s.add(_req("b", 4))
    o = s.schedule()
    assert o.num_scheduled_tokens == {"a": 10}
    s.update(o, {"a": [1]})
    o = s.schedule()                       # b's prefill, a is not decoded beside it
    assert o.num_scheduled_tokens == {"b": 4}
    s.update(o, {"b": [1]})
    assert s.schedule().num_scheduled_tokens == {"a": 1, "b": 1}


def test_restatement_is_causal_windowed_and_sink_sensitive():
    from oracle import pumopel_ref as R

    d = _cfg(window=3, layers=[_cfg(window=3)["layers"][0]])       # one attention layer: receptive field = the window
    W = random_weights(HybridConfig.from_dict(d), seed=1)
    t = torch.randint(0, 20, (12,), generator=torch.Generator().manual_seed(0)).tolist()
    full = R.forward(d, W, t)
    assert torch.allclose(R.forward(d, W, t[:7]), full[:7], atol=1e-12)                  # causal
    t2 = list(t)
    t2[8] = (t2[8] + 1) % 20
    moved = (R.forward(d, W, t2) - full).abs().amax(-1)
    assert moved[:8].max() == 0 and moved[8:11].min() > 0 and moved[11] == 0             # i sees j iff 0 <= i - j < 3
    W2 = dict(W)
    W2["l0.mix.sink"] = W["l0.mix.sink"] + 3.0
    assert (R.forward(d, W2, t) - full).abs().max() > 1e-3                               # the sink is in the denominator
