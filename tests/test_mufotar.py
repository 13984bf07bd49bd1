"""Mufotar on the CPU: the plain implementation's mechanisms one by one, configuration, builder, weights, cache and states, and
the engine's host side (step building, pages, state slots, scheduler) with the torch stand-in kernels, against the plain
implementation."""
import json
import math

import pytest
import torch

import plain_mufotar as plain
from mufotar_cases import CASES, check_long_decoding, check_mixed, check_whole_and_cut, plain_logits, setup_case
from torch_kernels import TorchKernels


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("mufotar")
    return {name: setup_case(tmp, name, "float32") for name in CASES}


D = torch.float64


# ------------------------------------------------------------------------------------------------ the plain implementation itself
def test_plain_layer_norm_has_a_bias_and_the_gelu_is_the_tanh_form():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=D)
    y = plain.layer_norm(x, torch.tensor([2.0, 2.0, 2.0, 2.0], dtype=D), torch.tensor([0.5, 0.0, 0.0, -1.0], dtype=D), 0.0)
    sd = math.sqrt((4 + 1 + 0 + 9) / 4)
    assert torch.allclose(y, torch.tensor([[-4 / sd + 0.5, -2 / sd, 0.0, 6 / sd - 1.0]], dtype=D))
    z = torch.tensor([0.7], dtype=D)
    assert plain.gelu_tanh(z).item() == pytest.approx(0.5 * 0.7 * (1 + math.tanh(math.sqrt(2 / math.pi) * (0.7 + 0.044715 * 0.7 ** 3))))


def test_plain_rotation_turns_the_first_entries_in_halves():
    x = torch.arange(12, dtype=D).view(1, 1, 12) + 1
    got = plain.rotate_half(x, torch.tensor([3]), 4, 10.0)[0, 0]
    a = 3 * torch.tensor([1.0, 10.0 ** -0.5], dtype=D)
    assert torch.allclose(got[[0, 2]], torch.stack([1 * a[0].cos() - 3 * a[0].sin(), 3 * a[0].cos() + 1 * a[0].sin()]))
    assert torch.allclose(got[[1, 3]], torch.stack([2 * a[1].cos() - 4 * a[1].sin(), 4 * a[1].cos() + 2 * a[1].sin()]))
    assert torch.equal(got[4:], x[0, 0, 4:])       # the rest passes


def test_plain_convolution_and_delta_rule_by_hand():
    u = torch.tensor([[1.0], [2.0], [3.0]], dtype=D)
    y = plain.causal_conv(u, torch.tensor([[10.0, 1.0]], dtype=D), torch.tensor([0.5], dtype=D))      # the last column is the current token's
    assert y.flatten().tolist() == [1.5, 12.5, 23.5]
    # the delta rule writes before it reads: with beta = 1, no decay and a unit key, reading with the key returns the value
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "conv": 2}
    one = torch.tensor([[0.0, 1.0]] * 2)
    W = {"p.q": torch.eye(2), "p.k": torch.eye(2), "p.v": torch.eye(2), "p.q.conv": one, "p.k.conv": one, "p.v.conv": one, "p.b": torch.full((1, 2), 50.0),
         "p.a": torch.zeros(1, 2), "p.dt_bias": torch.full((1,), -60.0), "p.A_log": torch.zeros(1), "p.g": torch.eye(2), "p.norm": torch.ones(2), "p.o": torch.eye(2)}
    W = {k: v.double() for k, v in W.items()}
    h = torch.tensor([[3.0, 0.0]], dtype=D)
    out = plain.delta_mixer(h, m, W, "p", 1e-12)
    # q = k = silu(3) e_0 made unit; v = silu(h); o = v (k . q) = v / sqrt(2); then the unit norm over vdim, times silu(h)
    v = plain.silu(h)
    assert torch.allclose(out, v / v.pow(2).mean().sqrt() * plain.silu(h), atol=1e-6)
    # a decay per head: two tokens, the second reads what is left of the first (beta 1, k the same unit vector: the write replaces it)
    W["p.dt_bias"] = torch.zeros(1, dtype=D)
    h2 = torch.tensor([[3.0, 0.0], [3.0, 0.0]], dtype=D)
    W["p.q.conv"] = W["p.k.conv"] = W["p.v.conv"] = one.double()
    out2 = plain.delta_mixer(h2, m, W, "p", 1e-12)
    assert torch.allclose(out2[1], out2[0], atol=1e-9)      # S k after the write is v again, whatever the decay was


def test_plain_selective_scan_by_hand():
    m = {"inner": 1, "state": 2, "dt_rank": 1, "conv": 1}
    W = {"p.in": torch.tensor([[1.0], [0.0]]), "p.conv": torch.tensor([[1.0]]), "p.conv.b": torch.zeros(1), "p.x": torch.tensor([[0.0], [1.0], [2.0], [1.0], [2.0]]),
         "p.dt": torch.tensor([[0.0]]), "p.dt.b": torch.tensor([math.log(math.e - 1)]), "p.A_log": torch.tensor([[0.0, math.log(2.0)]]), "p.D": torch.tensor([3.0]),
         "p.o": torch.tensor([[1.0]])}
    W = {k: v.double() for k, v in W.items()}
    h = torch.tensor([[1.0], [1.0]], dtype=D)
    out = plain.selective_scan(h, m, W, "p").flatten()
    x = plain.silu(torch.tensor(1.0, dtype=D)).item()           # after the one-tap convolution and SiLU; dt = softplus(ln(e - 1)) = 1
    S1 = [x * x, x * 2 * x]                                      # B = (x, 2x), C the same
    y1 = S1[0] * x + S1[1] * 2 * x + 3 * x
    S2 = [math.exp(-1) * S1[0] + x * x, math.exp(-2) * S1[1] + 2 * x * x]
    y2 = S2[0] * x + S2[1] * 2 * x + 3 * x
    assert out.tolist() == pytest.approx([y1 * 0.0, y2 * 0.0])  # z = 0: silu(z) = 0
    W["p.in"] = torch.tensor([[1.0], [1.0]], dtype=D)           # z = 1
    out = plain.selective_scan(h, m, W, "p").flatten()
    assert out.tolist() == pytest.approx([y1 * x, y2 * x])


def test_plain_router_correction_identity_and_weights():
    mlp = {"kind": "moe", "expert": {"ff": 1}, "router": {"experts": 2, "identity": 1, "top": 2}}
    W = {"p.router": torch.tensor([[2.0], [1.0], [0.0]]), "p.correction": torch.tensor([0.0, -1.0, 0.5]),
         "p.e0.gate": torch.tensor([[1.0]]), "p.e0.up": torch.tensor([[2.0]]), "p.e0.down": torch.tensor([[3.0]]),
         "p.e1.gate": torch.tensor([[9.0]]), "p.e1.up": torch.tensor([[9.0]]), "p.e1.down": torch.tensor([[9.0]])}
    W = {k: v.double() for k, v in W.items()}
    h = torch.tensor([[1.0]], dtype=D)
    s = torch.softmax(torch.tensor([2.0, 1.0, 0.0], dtype=D), 0)
    idx, w = plain.route(h, mlp, W, "p")
    assert sorted(idx[0].tolist()) == [0, 2]                    # the correction lifts the identity expert over expert 1 ...
    got = dict(zip(idx[0].tolist(), w[0].tolist()))
    assert got[0] == pytest.approx((s[0] / (s[0] + s[2])).item()) and got[2] == pytest.approx((s[2] / (s[0] + s[2])).item())   # ... but is not in the weights
    y = plain.experts(h, mlp, W, "p")[0, 0].item()
    e0 = plain.silu(torch.tensor(1.0, dtype=D)).item() * 2.0 * 3.0
    assert y == pytest.approx(got[0] * e0 + got[2] * 1.0)       # the identity expert returns the input
    mlp["shared"] = {"ff": 1}
    W.update({"p.shared.gate": torch.tensor([[1.0]], dtype=D), "p.shared.up": torch.tensor([[1.0]], dtype=D), "p.shared.down": torch.tensor([[-2.0]], dtype=D)})
    assert plain.experts(h, mlp, W, "p")[0, 0].item() == pytest.approx(y - 2.0 * plain.silu(torch.tensor(1.0, dtype=D)).item())


def test_plain_both_sublayers_read_the_same_norm_and_the_logits_are_capped(cases):
    folder, cfg, tensors, prompts, want = cases["A"]
    layers = []
    logits = plain.forward(cfg, tensors, prompts["d"], D, layers)
    assert len(layers) == len(cfg["layers"]) and float(logits.abs().max()) < cfg["logit_softcap"]
    t = {k: v.double() for k, v in tensors.items()}
    x0 = t["embed"][torch.tensor(prompts["d"])]
    h = plain.layer_norm(x0, t["l0.norm1"], t["l0.norm1.b"], cfg["norm"]["eps"])
    x1 = x0 + plain.delta_mixer(h, cfg["layers"][0]["mixer"], t, "l0.mix", cfg["norm"]["eps"]) + plain.feed_forward(h, cfg["layers"][0]["mlp"], t, "l0.mlp")
    assert torch.allclose(layers[0], x1)


# ------------------------------------------------------------------------------------------------ configuration, builder, cache
def test_config_reads_every_key():
    from llm_infrence_engine_b200.config import ConfigError
    from llm_infrence_engine_b200.config.model_config import MufotarConfig, RoutedExpertsConfig

    cfg = MufotarConfig.from_dict(CASES["A"][0])
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.logit_softcap) == (83, 48, 1e-5, 12.0) and len(cfg.layers) == 5
    d, p, e = cfg.layers[0], cfg.layers[1], cfg.layers[2]
    assert d.kind == "delta" and (d.mixer.heads, d.mixer.kv_heads, d.mixer.dim, d.mixer.vdim, d.mixer.conv, d.mlp) == (4, 2, 16, 24, 3, 64)
    assert (p.mixer.left.heads, p.mixer.left.kv_heads, p.mixer.left.dim, p.mixer.left.vdim, p.mixer.left.scale, p.mixer.left.qk_norm) == (6, 2, 24, 16, 0.2, True)
    assert (p.mixer.left.rot.dims, p.mixer.left.rot.base, p.mixer.left.rot.factor, p.mixer.left.mask_size, p.mixer.left.interleaved) == (16, 1000.0, None, None, False)
    assert (p.mixer.right.inner, p.mixer.right.state, p.mixer.right.dt_rank, p.mixer.right.conv, p.mixer.left_scale, p.mixer.right_scale) == (40, 12, 5, 4, 0.7, 1.3)
    assert p.mlp == RoutedExpertsConfig(5, 2, 3, 24, 40) and e.mlp is None
    assert [layer.weights_of for layer in cfg.layers] == [None, None, None, 1, 0]
    b = MufotarConfig.from_dict(CASES["B"][0])
    assert b.logit_softcap is None and b.layers[0].mlp == RoutedExpertsConfig(3, 0, 1, 32, None) and b.layers[2].mixer.left.rot is None
    assert MufotarConfig.from_dict(CASES["C"][0]).layers[0].weights_of == 2
    for change in (lambda c: c["layers"][3].update(weights_of=4), lambda c: c["layers"][3]["mixer"]["left"].update(heads=3),
                   lambda c: c["layers"][0].update(type="convolution"), lambda c: c["layers"][1]["mlp"]["router"].update(top=8),
                   lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=26), lambda c: c["layers"][1]["mixer"].pop("left_scale"),
                   lambda c: c["layers"][0]["mlp"].update(kind="sparse"), lambda c: c.update(logit_softcap=-1.0)):
        bad = json.loads(json.dumps(CASES["A"][0]))
        change(bad)
        with pytest.raises(ConfigError):
            MufotarConfig.from_dict(bad)


def test_builder_names_the_checkpoint_tensors_and_the_cache():
    from llm_infrence_engine_b200.cache.spec import FixedStateSpec, PagedKVSpec
    from llm_infrence_engine_b200.engine.step import group_layout, has_fixed_state
    from llm_infrence_engine_b200.models import build_model_spec
    from llm_infrence_engine_b200.weights.loader import expected_tensors

    spec = build_model_spec(CASES["A"][0])
    names = set(expected_tensors(spec))
    assert {"embed", "final.norm", "final.norm.b", "l0.norm1", "l0.norm1.b", "l0.mix.q", "l0.mix.q.conv", "l0.mix.k.conv", "l0.mix.v.conv", "l0.mix.b", "l0.mix.a",
            "l0.mix.g", "l0.mix.A_log", "l0.mix.dt_bias", "l0.mix.norm", "l0.mix.o", "l0.mlp.gate", "l0.mlp.up", "l0.mlp.down", "l1.mix.left.q", "l1.mix.left.k",
            "l1.mix.left.v", "l1.mix.left.o", "l1.mix.left.q.norm", "l1.mix.left.k.norm", "l1.mix.right.in", "l1.mix.right.conv", "l1.mix.right.conv.b",
            "l1.mix.right.x", "l1.mix.right.dt", "l1.mix.right.dt.b", "l1.mix.right.A_log", "l1.mix.right.D", "l1.mix.right.o", "l1.mlp.router", "l1.mlp.correction",
            "l1.mlp.e0.gate", "l1.mlp.e4.down", "l1.mlp.shared.up", "l2.mix.q"} <= names
    assert not any(n.startswith(("l3.", "l4.", "l2.mlp", "l1.mlp.e5", "head", "l0.norm2", "l1.mix.left.q.conv")) for n in names)
    assert expected_tensors(spec)["l1.mix.right.A_log"][0] == (40, 12) and expected_tensors(spec)["l1.mlp.router"][0] == (7, 48)
    # a layer that runs on another's weights is that layer's part once more, with a cache entry of its own
    assert [(c.layer, c.cache, c.write) for c in spec.schedule] == [(0, 0, True), (1, 1, True), (2, 2, True), (1, 3, True), (0, 4, True)]
    specs = spec.cache_specs()
    assert specs[0] == (FixedStateSpec((4, 24, 16)), FixedStateSpec((2, 2 * 2 * 16 + 4 * 24))) == specs[4]
    assert specs[1] == (PagedKVSpec(2, 24, None, 16, 0, None), (FixedStateSpec((40, 12)), FixedStateSpec((3, 40)))) == specs[3]
    groups, of_entry = group_layout(specs)
    assert len(groups) == 1 and of_entry == [(None, None), (0, (None, None)), (None, None), (0, (None, None)), (None, None)]
    assert has_fixed_state(specs)
    later = build_model_spec(CASES["C"][0])     # the first layer runs on the weights of the third
    assert [(c.layer, c.cache) for c in later.schedule] == [(1, 0), (0, 1), (1, 2)] and "l0.mix.q" not in expected_tensors(later)


def test_weights_load_experts_stacked_and_sections_on_16_byte_columns(tmp_path):
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
    delta, pair, ff = spec.layers[0].mixer, spec.layers[1].mixer, spec.layers[1].ff
    assert delta.w_in.shape[0] % 8 == 0 and delta.b_col % 8 == 0 and delta.a_col % 8 == 0 and delta.g_col % 8 == 0
    assert torch.equal(delta.w_in[delta.a_col:delta.a_col + 4], t["l0.mix.a"]) and torch.equal(delta.w_in[delta.g_col:delta.g_col + 96], t["l0.mix.g"])
    assert torch.equal(delta.w_in[delta.b_col:delta.b_col + 4], t["l0.mix.b"]) and delta.conv_w.shape == (2 * 32 + 96, 3)
    assert pair.scales == (0.7, 1.3) and not pair.params() and pair.left.qk_norm and pair.left.position.dims == 16
    scan = pair.right
    assert scan.w_x.shape == (32, 40) and scan.w_dt.shape == (40, 32)       # 5 + 2 * 12 = 29 rows padded to 32; zero columns beside the rank
    assert torch.equal(scan.w_dt[:, :5], t["l1.mix.right.dt"]) and float(scan.w_dt[:, 5:].abs().max()) == 0.0
    assert ff.w_gate_up.shape == (5, 48, 48) and ff.w_down.shape == (5, 48, 24) and ff.shared.w_gate_up.shape == (80, 48)
    assert torch.equal(ff.w_gate_up[3, :24], t["l1.mlp.e3.gate"]) and torch.equal(ff.w_gate_up[3, 24:], t["l1.mlp.e3.up"]) and torch.equal(ff.w_down[4], t["l1.mlp.e4.down"])
    assert spec.head.matrix() is spec.embedding.table and spec.head.softcap == 12.0 and spec.final_norm.bias is not None
    assert spec.layers[2].ff is None


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
