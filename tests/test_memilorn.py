"""Memilorn on the CPU: the plain implementation's mechanisms one by one, configuration, builder, weights, cache and states, and
the engine's host side (step building, pages, state slots, scheduler) with the torch stand-in kernels, against the plain
implementation."""
import json
import math

import pytest
import torch

import plain_memilorn as plain
from memilorn_cases import CASES, check_long_decoding, check_mixed, check_whole_and_cut, plain_logits, setup_case
from torch_kernels import TorchKernels


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("memilorn")
    return {name: setup_case(tmp, name, "float32") for name in CASES}


D = torch.float64


# ------------------------------------------------------------------------------------------------ the plain implementation itself
def test_plain_layer_norm_has_no_bias_and_the_variance_is_about_the_mean():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=D)
    w = torch.tensor([1.0, 2.0, 0.5, 1.0], dtype=D)
    var = ((x - 3.0) ** 2).mean()
    assert torch.allclose(plain.layer_norm(x, w, 1e-3), (x - 3.0) / math.sqrt(float(var) + 1e-3) * w)


def test_plain_matrix_memory_by_hand():
    """Two tokens, one head, written out: the maximum starts at 0 (not at minus infinity), so a first token with a negative input
    gate is taken in with exp(i) < 1, and the denominator is bounded below by exp(-m)."""
    q = torch.tensor([[1.0, 0.0], [0.5, 0.5]], dtype=D)
    k = torch.tensor([[2.0, 1.0], [1.0, -1.0]], dtype=D)
    v = torch.tensor([[3.0], [5.0]], dtype=D)
    i_log, f_log = torch.tensor([-1.0, 2.0], dtype=D), torch.tensor([-0.5, -0.25], dtype=D)
    o = plain.matrix_memory_cell(q, k, v, i_log, f_log)
    # token 0: m = max(-0.5 + 0, -1) = -0.5; S = e^(-1 + 0.5) k0 v0^T; n = e^(-0.5) k0; den = max(|n . q0|, e^0.5) + 1e-6
    b0 = math.exp(-0.5)
    o0 = b0 * 2.0 * 3.0 / (max(abs(b0 * 2.0), math.exp(0.5)) + 1e-6)
    assert abs(float(o[0, 0]) - o0) < 1e-12
    # token 1: m = max(-0.25 - 0.5, 2) = 2; S = e^(-0.75 - 2) S + e^0 k1 v1^T
    a1 = math.exp(-0.25 - 0.5 - 2.0)
    S = a1 * b0 * torch.outer(k[0], v[0]) + torch.outer(k[1], v[1])
    n = a1 * b0 * k[0] + k[1]
    o1 = float(S.T @ q[1]) / (max(abs(float(n @ q[1])), math.exp(-2.0)) + 1e-6)
    assert abs(float(o[1, 0]) - o1) < 1e-12


def test_plain_rotation_turns_neighbouring_pairs_of_the_first_entries():
    x = torch.arange(1.0, 7.0, dtype=D).view(1, 1, 6).repeat(3, 1, 1)
    y = plain.rotate_neighbours(x, torch.arange(3), 4, 100.0)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 4:], x[..., 4:])          # position 0 and the entries beyond dims pass
    a0, a1 = 2.0 * 1.0, 2.0 * 100.0 ** (-2.0 / 4)
    assert abs(float(y[2, 0, 0]) - (1 * math.cos(a0) - 2 * math.sin(a0))) < 1e-12 and abs(float(y[2, 0, 1]) - (2 * math.cos(a0) + 1 * math.sin(a0))) < 1e-12
    assert abs(float(y[2, 0, 2]) - (3 * math.cos(a1) - 4 * math.sin(a1))) < 1e-12


def test_plain_sink_joins_the_denominator_once_and_heads_are_mixed_before_the_mask():
    s = torch.tensor([[[0.0, -math.inf], [1.0, 2.0]]], dtype=D)
    p = plain.sink_softmax(s, torch.tensor([0.5], dtype=D))
    assert abs(float(p[0, 0, 0]) - 1.0 / (1.0 + math.exp(0.5))) < 1e-12 and float(p[0, 0, 1]) == 0.0
    assert abs(float(p[0, 1].sum()) - (math.e + math.e ** 2) / (math.e + math.e ** 2 + math.exp(0.5))) < 1e-12
    # one token, two heads on one key/value head: with q = k the scores are |k|^2 * scale for both; the mix makes head 0 see 1.5 times it
    m = {"heads": 2, "kv_heads": 1, "dim": 2, "vdim": 1, "scale": 0.5}
    t = {"x.q": torch.tensor([[1.0, 0], [0, 1], [1, 0], [0, 1]], dtype=D), "x.k": torch.eye(2, dtype=D), "x.v": torch.tensor([[1.0, 1.0]], dtype=D),
         "x.talk": torch.tensor([[1.0, 0.5], [0.0, 1.0]], dtype=D), "x.sink": torch.tensor([0.0, 0.0], dtype=D), "x.g": torch.zeros(2, 2, dtype=D),
         "x.o": torch.eye(2, dtype=D)}
    h = torch.tensor([[1.0, 2.0]], dtype=D)
    out = plain.talking_attention(h, m, t, "x")
    s0 = 0.5 * 5.0
    want = [0.5 * 3.0 * math.exp(1.5 * s0) / (math.exp(1.5 * s0) + 1.0), 0.5 * 3.0 * math.exp(s0) / (math.exp(s0) + 1.0)]
    assert torch.allclose(out[0], torch.tensor(want, dtype=D))


def test_plain_router_weighs_the_inputs_and_does_not_renormalise():
    t = {"m.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [-1.0, 0.0]], dtype=D)}
    for e in range(3):
        t[f"m.e{e}.gate"] = torch.full((1, 2), 0.5 + e, dtype=D)
        t[f"m.e{e}.up"] = torch.full((1, 2), 0.25, dtype=D)
        t[f"m.e{e}.down"] = torch.ones(2, 1, dtype=D)
    mlp = {"router": {"experts": 3, "top": 2}, "expert": {"ff": 1, "limit": 1.0}}
    h = torch.tensor([[2.0, 1.0]], dtype=D)
    idx, w = plain.route(h, mlp, t, "m")
    assert idx.tolist() == [[0, 1]] and torch.allclose(w, torch.sigmoid(torch.tensor([[2.0, 1.0]], dtype=D)))
    out = plain.experts(h, mlp, t, "m")
    total = 0.0
    for e, s in zip((0, 1), w[0].tolist()):
        g = min((0.5 + e) * 3.0 * s, 1.0)                    # the score is on the input, and the gate is bounded from above only
        u = max(min(0.25 * 3.0 * s, 1.0), -1.0)
        total += g / (1.0 + math.exp(-1.702 * g)) * (u + 1.0)
    assert torch.allclose(out, torch.full((1, 2), total, dtype=D))


def test_plain_running_order_loops_and_adds_the_embedding_again(cases):
    assert plain.running_order(CASES["A"][0]) == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert plain.running_order(CASES["B"][0]) == [(0, False), (1, False), (2, False)]
    assert plain.running_order(CASES["C"][0]) == [(0, False), (1, False), (0, True), (1, False), (2, False)]
    folder, cfg, tensors, prompts, want = cases["C"]
    runs = []
    plain.forward(cfg, tensors, prompts["d"], D, layers_out=runs)
    assert len(runs) == 5
    # without the embedding added before the second pass the result differs
    other = {k: v.clone() for k, v in tensors.items()}
    no_loop = json.loads(json.dumps(cfg))
    no_loop["loop"]["times"] = 1
    assert not torch.allclose(plain.forward(no_loop, other, prompts["d"], D), want["d"])


# ------------------------------------------------------------------------------------------------ configuration, builder, weights
def test_config_reads_every_key():
    from llm_infrence_engine_b200.config import ConfigError, MemilornConfig
    from llm_infrence_engine_b200.config.model_config import SigmoidExpertsConfig

    cfg = MemilornConfig.from_dict(CASES["A"][0])
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.loop_start, cfg.loop_stop, cfg.loop_times) == (83, 48, 1e-5, 1, 3, 3) and len(cfg.layers) == 4
    a, m, l, last = cfg.layers
    assert a.kind == "attention" and (a.mixer.heads, a.mixer.kv_heads, a.mixer.dim, a.mixer.vdim, a.mixer.scale, a.mixer.softcap) == (6, 2, 16, 8, 0.3, 5.0)
    assert (a.mixer.rot.dims, a.mixer.rot.base) == (8, 100.0)
    assert m.kind == "mlstm" and (m.mixer.heads, m.mixer.dim, m.mixer.vdim, m.mixer.gate_cap) == (3, 8, 16, 4.0)
    assert l.kind == "latent_attention" and (l.mixer.heads, l.mixer.dim, l.mixer.vdim, l.mixer.kv_rank, l.mixer.scale) == (4, 8, 12, 16, 0.4)
    assert a.mlp == SigmoidExpertsConfig(5, 2, 24, 1.5, 40, 2.5) and l.mlp == SigmoidExpertsConfig(4, 3, 16, 3.0, None, 0.0) and last.mlp is None
    assert [r[0] for r in cfg.running_order()] == [0, 1, 2, 1, 2, 1, 2, 3] and [r[2] for r in cfg.running_order()] == [False, False, False, True, False, True, False, False]
    b = MemilornConfig.from_dict(CASES["B"][0])
    assert (b.loop_start, b.loop_stop, b.loop_times) == (0, 0, 1) and b.layers[1].mixer.softcap is None and b.layers[2].mixer.gate_cap is None
    assert MemilornConfig.from_dict(CASES["C"][0]).layers[1].mixer.rot is None
    for change in (lambda c: c["loop"].update(stop=5), lambda c: c["loop"].update(start=3, stop=2), lambda c: c["loop"].update(times=0),
                   lambda c: c["layers"][0]["mixer"].update(heads=5), lambda c: c["layers"][0].update(type="convolution"),
                   lambda c: c["layers"][0]["mlp"]["router"].update(top=6), lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18),
                   lambda c: c["layers"][0]["mlp"].update(kind="dense"), lambda c: c["layers"][1]["mixer"].update(gate_cap=-1.0),
                   lambda c: c["layers"][0]["mlp"]["expert"].update(limit=0.0), lambda c: c["layers"][2]["mixer"].pop("kv_rank"), lambda c: c["norm"].update(eps=0.0)):
        bad = json.loads(json.dumps(CASES["A"][0]))
        change(bad)
        with pytest.raises(ConfigError):
            MemilornConfig.from_dict(bad)


def test_builder_names_the_checkpoint_tensors_and_the_cache():
    from llm_infrence_engine_b200.cache.spec import FixedStateSpec, PagedKVSpec
    from llm_infrence_engine_b200.engine.step import group_layout, has_fixed_state
    from llm_infrence_engine_b200.models import build_model_spec
    from llm_infrence_engine_b200.weights.loader import expected_tensors

    spec = build_model_spec(CASES["A"][0])
    want = expected_tensors(spec)
    names = set(want)
    assert {"embed", "final.norm", "l0.norm1", "l0.norm2", "l0.ls1", "l0.ls2", "l0.mix.q", "l0.mix.k", "l0.mix.v", "l0.mix.g", "l0.mix.talk", "l0.mix.sink", "l0.mix.o",
            "l0.mlp.router", "l0.mlp.e0.gate", "l0.mlp.e4.down", "l0.mlp.shared.up", "l1.mix.q", "l1.mix.k", "l1.mix.v", "l1.mix.g", "l1.mix.o", "l1.mix.norm", "l1.mix.i",
            "l1.mix.i.b", "l1.mix.f", "l1.mix.f.b", "l2.mix.q", "l2.mix.dkv", "l2.mix.dkv.norm", "l2.mix.uk", "l2.mix.uv", "l2.mix.g", "l2.mix.o", "l3.ls1"} <= names
    assert not any(n.startswith(("l4.", "l3.mlp", "l3.norm2", "l3.ls2", "l2.mlp.shared", "l0.mlp.e5", "l0.mlp.correction", "head", "l2.mix.dq", "l2.mix.sink", "final.norm.b")) for n in names)
    assert want["l0.mix.g"][0] == (6, 48) and want["l0.mix.talk"][0] == (6, 6) and want["l2.mix.g"][0] == (4, 48) and want["l1.mix.g"][0] == (48, 48)
    assert want["l1.mix.norm"][0] == (48,) and want["l2.mix.uk"][0] == (32, 16) and want["l2.mix.uv"][0] == (48, 16) and want["l0.mlp.router"][0] == (5, 48)
    # every run of a looped layer is that layer's part once more with a cache entry of its own; further passes open with the embedding
    assert [(c.layer, c.cache, c.add_embedding) for c in spec.schedule] == [(0, 0, False), (1, 1, False), (2, 2, False), (1, 3, True), (2, 4, False),
                                                                          (1, 5, True), (2, 6, False), (3, 7, False)]
    specs = spec.cache_specs()
    assert specs[0] == PagedKVSpec(2, 16, None, 8, 0, None)
    assert specs[1] == (FixedStateSpec((3, 17, 8)), FixedStateSpec((3,))) == specs[3] == specs[5]
    assert specs[2] == PagedKVSpec(1, 16, None, 0) == specs[4] == specs[6] and specs[7] == (FixedStateSpec((2, 13, 12)), FixedStateSpec((2,)))
    groups, of_entry = group_layout(specs)
    assert len(groups) == 2 and of_entry == [0, (None, None), 1, (None, None), 1, (None, None), 1, (None, None)]
    assert has_fixed_state(specs)
    assert [(c.layer, c.add_embedding) for c in build_model_spec(CASES["C"][0]).schedule] == [(0, False), (1, False), (0, True), (1, False), (2, False)]


def test_weights_load_into_joined_projections_and_stacked_experts(tmp_path):
    from llm_infrence_engine_b200.models import build_model_spec
    from llm_infrence_engine_b200.weights import load_weights
    from llm_infrence_engine_b200.weights.random_init import random_tensors
    from llm_infrence_engine_b200.weights.safetensors_io import write_safetensors

    cfg = CASES["A"][0]
    t = random_tensors(cfg, 1)
    (tmp_path / "m").mkdir()
    write_safetensors(tmp_path / "m" / "model.safetensors", {k: v.contiguous() for k, v in t.items()})
    spec = build_model_spec(cfg)
    load_weights(spec, tmp_path / "m", torch.float32, "cpu")
    att, mem, lat = spec.layers[0].mixer, spec.layers[1].mixer, spec.layers[2].mixer
    assert att.w_qkv.shape == (6 * 16 + 2 * 16 + 2 * 8 + 8, 48) and torch.equal(att.w_qkv[att.channels:att.channels + 6], t["l0.mix.g"])   # 6 gate rows padded to 8
    assert att.talk.shape == (6, 6) and att.sink.shape == (6,) and att.interleaved and att.softcap == 5.0 and att.position.dims == 8
    assert (mem.q_col, mem.k_col, mem.v_col, mem.g_col) == (0, 24, 48, 96) and mem.w_in.shape == (144, 48) and mem.w_gates.shape == (8, 48)
    assert torch.equal(mem.w_gates[:3], t["l1.mix.i"]) and torch.equal(mem.w_gates[3:6], t["l1.mix.f"]) and float(mem.w_gates[6:].abs().max()) == 0.0
    assert lat.q_rank == 0 and lat.w_q.shape == (32, 48) and lat.w_in.shape == (24, 48) and lat.g_col == 16 and torch.equal(lat.w_in[16:20], t["l2.mix.g"])
    ff = spec.layers[0].ff
    assert ff.w_gate_up.shape == (5, 48, 48) and ff.w_down.shape == (5, 48, 24) and ff.shared.w_gate_up.shape == (80, 48) and ff.correction is None
    assert torch.equal(ff.w_gate_up[3, :24], t["l0.mlp.e3.gate"]) and torch.equal(ff.w_gate_up[3, 24:], t["l0.mlp.e3.up"])
    assert (ff.scoring, ff.weight_inputs, ff.expert_glu, ff.shared.limit) == ("sigmoid", True, (1.5, 1.702, 1.0), 2.5)
    assert torch.equal(spec.layers[1].scale1, t["l1.ls1"]) and torch.equal(spec.layers[1].scale2, t["l1.ls2"]) and spec.layers[3].scale2 is None
    assert spec.head.matrix() is spec.embedding.table and spec.final_norm.bias is None and spec.layers[3].ff is None


# ------------------------------------------------------------------------------------------------ the engine's host side
@pytest.mark.parametrize("name", sorted(CASES))
def test_engine_whole_and_cut_on_cpu(cases, name):
    check_whole_and_cut(cases[name], name, "float32", TorchKernels(), "cpu", only=("b", "c", "d", "f"))


def test_engine_mixed_batches_on_cpu(cases):
    check_mixed(cases["A"], "A", "float32", TorchKernels(), "cpu", seeds=(0,))


def test_engine_long_decoding_on_cpu(cases):
    check_long_decoding(cases["B"], "B", "float32", TorchKernels(), "cpu", total=90)


def test_greedy_generation_through_the_entry_point_on_cpu(cases):
    from llm_infrence_engine_b200.engine import Engine

    folder, cfg, tensors, prompts, want = cases["C"]
    eng = Engine(folder, kernels=TorchKernels(), dtype="float32", device="cpu", max_len=128, max_seqs=3, block_size=4, num_blocks=80,
                 max_num_batched_tokens=24)
    ps = [prompts["c"], prompts["d"], prompts["f"], prompts["b"][:30]]
    results = eng.generate(ps, max_new_tokens=8)
    for p, r in zip(ps, results):
        seq = list(p) + r.token_ids
        ref = plain_logits(cfg, tensors, seq)[len(p) - 1:-1]
        assert r.token_ids == ref.argmax(-1).tolist()
    eng.cache.check_invariants()
    assert all(pool.num_free == pool.capacity for pool in eng.cache.pools)
