"""Mufotar on the GPU: every new kernel against its plain torch statement, and the engine (both dtypes) against the plain
implementation: whole prompts, decoding token by token, portions down to two tokens, mixed batches on reused pages and state
slots, long decoding, greedy generation through the entry point, decode steps from CUDA graphs, and inputs made so that a far
key, a lost state, a wrong expert or a forgotten identity expert shows in the result."""
from types import SimpleNamespace

import pytest
import torch

from mufotar_cases import (CASES, check_long_decoding, close_calls, check_mixed, check_whole_and_cut, cuts_of, load_plain, make_folder, plain_logits, prompt,
                           replayer, row_errors, run_alone, setup_case)
from torch_kernels import TorchKernels

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def K():
    from llm_infrence_engine_b200.csrc import get_kernels

    return get_kernels()


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("mufotar")
    return {(name, dtype): setup_case(tmp, name, dtype) for name in CASES for dtype in DTYPES}


def close(got, want, dtype, what, scale=None, f32=4e-6):
    tol = (f32 if dtype == "float32" else 1.2e-2) * max(1.0, float(want.float().abs().max()) if scale is None else scale)
    err = float((got.float().cpu() - want.float().cpu()).abs().max())
    assert err <= tol, f"{what} ({dtype}): {err:.3g} > {tol:.3g}"


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def ragged(lens, slots):
    """The description of a step whose requests bring ``lens`` rows and own the state rows ``slots``: for the CPU and for the GPU."""
    starts = [0]
    for n in lens:
        starts.append(starts[-1] + n)
    host = SimpleNamespace(seq_starts_dev=torch.tensor(starts, dtype=torch.int32), seq_slots=torch.tensor(slots, dtype=torch.int32),
                           num_seqs=len(lens), max_seq_len=max(lens), seq_lens=list(lens), _tables={})
    dev = SimpleNamespace(**{**host.__dict__, "seq_starts_dev": host.seq_starts_dev.cuda(), "seq_slots": host.seq_slots.cuda(), "_tables": {}})
    return host, dev


# ---------------------------------------------------------------------------------------------------------------------
# kernels

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C,NS,lens", [(392, 24, [37, 1, 9]), (100, 12, [3, 70]), (64, 16, [1, 1, 1]), (520, 64, [130]), (48, 130, [20, 5]), (36, 1, [2, 1]),
                                       (8, 256, [1, 33])])
def test_selective_scan(K, dtype, C, NS, lens):
    ref, T = TorchKernels(), TD[dtype]
    N = sum(lens)
    host, dev = ragged(lens, list(range(1, len(lens) + 1)))
    pad = 8
    x, dt = rnd(N, C, seed=1).to(T), rnd(N, C, seed=2).to(T)
    bc, z = rnd(N, pad + 2 * NS + 3, seed=3).to(T), rnd(N, 2 * C, seed=4).to(T)
    A_log = torch.log(0.5 + 3 * torch.rand(C, NS, generator=torch.Generator().manual_seed(5)))
    dt_bias, skip = rnd(C, seed=6, scale=0.5) - 2, rnd(C, seed=7)
    st = rnd(5, C, NS, seed=8, scale=0.3)
    st_dev = st.clone().cuda()
    want = ref.selective_scan(x, dt, bc, pad, pad + NS, z, C, A_log, dt_bias, skip, st, host)
    got = K.selective_scan(x.cuda(), dt.cuda(), bc.cuda(), pad, pad + NS, z.cuda(), C, A_log.cuda(), dt_bias.cuda(), skip.cuda(), st_dev, dev)
    close(got, want, dtype, "selective_scan")
    close(st_dev, st, "float32", "selective_scan's states", f32=2e-5)
    assert torch.equal(st_dev[0].cpu(), rnd(5, C, NS, seed=8, scale=0.3)[0])       # a row that no request owns is not touched


def test_selective_scan_carries_its_state_whatever_the_cut(K):
    """Whole, in two portions and token by token from the same start: the same bits (a channel's walk over its rows is one order)."""
    C, NS, N = 72, 24, 45
    x, dt, bc, z = rnd(N, C, seed=1), rnd(N, C, seed=2), rnd(N, 2 * NS, seed=3), rnd(N, C, seed=4)
    A_log, dt_bias, skip = rnd(C, NS, seed=5, scale=0.3), rnd(C, seed=6) - 1, rnd(C, seed=7)
    args = lambda lo, hi: (x[lo:hi].cuda(), dt[lo:hi].cuda(), bc[lo:hi].cuda(), 0, NS, z[lo:hi].cuda(), 0, A_log.cuda(), dt_bias.cuda(), skip.cuda())
    start = rnd(3, C, NS, seed=9)
    st = start.clone().cuda()
    whole = K.selective_scan(*args(0, N), st, ragged([N], [2])[1])
    for sizes in ([30, 15], [1] * N, [2] * 22 + [1]):
        st2 = start.clone().cuda()
        outs = [K.selective_scan(*args(lo, hi), st2, ragged([hi - lo], [2])[1]) for lo, hi in cuts_of(N, sizes)]
        assert torch.equal(torch.cat(outs), whole) and torch.equal(st2, st), f"portions of {sizes[:2]}"
    assert torch.equal(st[:2].cpu(), start[:2])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,DV,lens", [(4, 2, 32, 64, [23, 1, 5]), (3, 1, 10, 6, [40]), (6, 3, 128, 33, [2, 9]), (2, 2, 256, 16, [1, 1]), (5, 5, 24, 40, [70])])
def test_delta_rule_with_a_decay_per_head(K, dtype, H, G, D, DV, lens):
    ref, T = TorchKernels(), TD[dtype]
    N = sum(lens)
    host, dev = ragged(lens, list(range(len(lens))))
    qkv, z = rnd(N, 2 * G * D + H * DV, seed=1).to(T), rnd(N, 3 * H + 5, seed=2).to(T)
    A_log = torch.log(0.5 + 3 * torch.rand(H, generator=torch.Generator().manual_seed(3)))
    dt_bias = rnd(H, seed=4)
    st = rnd(4, H, DV, D, seed=5, scale=0.3)
    st_dev = st.clone().cuda()
    want = ref.delta_rule(qkv, H, G, D, DV, z[:, H + 1:2 * H + 1], z, 1, A_log, dt_bias, st, host, decay_per_head=True)
    zd = z.cuda()
    got = K.delta_rule(qkv.cuda(), H, G, D, DV, zd[:, H + 1:2 * H + 1], zd, 1, A_log.cuda(), dt_bias.cuda(), st_dev, dev, decay_per_head=True)
    close(got, want, "float32", "delta_rule", f32=2e-4)
    close(st_dev, st, "float32", "delta_rule's states", f32=2e-4)


def test_delta_rule_reads_back_a_far_write(K):
    """One token writes a value under a key that no later token's key touches, with decay 1 (a step size of zero); 400 tokens
    later a query along that key reads the value back; with a decay below 1 it reads the value times decay^400."""
    H, D, DV, N = 2, 16, 8, 402
    qkv = torch.zeros(N, 2 * H * D + H * DV)
    k0, v0 = torch.zeros(D), torch.arange(1.0, DV + 1)
    k0[3] = 50.0                                                             # made a unit vector by the kernel
    for h in range(H):
        qkv[0, H * D + h * D:H * D + (h + 1) * D] = k0
        qkv[0, 2 * H * D + h * DV:2 * H * D + (h + 1) * DV] = v0 * (h + 1)
        qkv[1:N - 1, H * D + h * D + 7] = 1.0                                # the keys between lie along another axis
        qkv[N - 1, h * D:(h + 1) * D] = k0                                   # the last query asks along the first key
        qkv[N - 1, H * D + h * D + 9] = 1.0
    beta = torch.full((N, H), 30.0)                                          # sigmoid(30) = 1: the write is whole
    for rate, keeps in ((-100.0, 1.0), (-4.0, None)):
        a = torch.full((N, H), rate)                                         # softplus(-100) = 0: no decay at all
        A_log, dt_bias = torch.zeros(H), torch.zeros(H)
        st = torch.zeros(2, H, DV, D).cuda()
        _, dev = ragged([N], [1])
        out = K.delta_rule(qkv.cuda(), H, H, D, DV, a.cuda(), beta.cuda(), 0, A_log.cuda(), dt_bias.cuda(), st, dev, decay_per_head=True).cpu()
        keeps = keeps if keeps is not None else float(torch.exp(-torch.nn.functional.softplus(torch.tensor(rate, dtype=torch.float64)) * (N - 1)))
        for h in range(H):
            want = v0 * (h + 1) * D ** -0.5 * keeps
            assert torch.allclose(out[N - 1, h * DV:(h + 1) * DV], want, rtol=2e-4, atol=1e-6), (rate, h)
        # the same, the last token alone from the state that the first 401 left
        st2 = torch.zeros(2, H, DV, D).cuda()
        K.delta_rule(qkv[:N - 1].cuda(), H, H, D, DV, a[:N - 1].cuda(), beta[:N - 1].cuda(), 0, A_log.cuda(), dt_bias.cuda(), st2, ragged([N - 1], [1])[1], decay_per_head=True)
        last = K.delta_rule(qkv[N - 1:].cuda(), H, H, D, DV, a[N - 1:].cuda(), beta[N - 1:].cuda(), 0, A_log.cuda(), dt_bias.cuda(), st2, ragged([1], [1])[1], decay_per_head=True)
        assert torch.allclose(last.cpu()[0], out[N - 1], rtol=1e-5, atol=1e-7) and torch.allclose(st2, st, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("dtype", DTYPES)
def test_layernorm_with_bias_gated_norm_pair_cap_and_gelu_unit(K, dtype):
    ref, T = TorchKernels(), TD[dtype]
    for N, Hd in ((1, 8), (37, 256), (5, 44), (130, 1000)):
        x, w, b = rnd(N, Hd, seed=1) + 0.5, 1 + rnd(Hd, seed=2, scale=0.2), rnd(Hd, seed=3)
        close(K.layernorm(x.cuda(), w.cuda(), 1e-6, T, bias=b.cuda()), ref.layernorm(x, w, 1e-6, T, bias=b), dtype, "layernorm with bias")
        rows = torch.tensor([N - 1, 0], dtype=torch.int32)
        close(K.layernorm(x.cuda(), w.cuda(), 1e-6, T, rows.cuda(), bias=b.cuda()), ref.layernorm(x, w, 1e-6, T, rows, bias=b), dtype, "layernorm of rows with bias")
    for N, Hh, DV, col in ((11, 4, 64, 8), (3, 3, 6, 0), (70, 2, 40, 16)):
        o, g, nw = rnd(N, Hh * DV, seed=4, scale=2.0), rnd(N, Hh * DV + col + 3, seed=5).to(T), 1 + rnd(DV, seed=6, scale=0.2)
        got = K.group_rmsnorm_gate(o.cuda(), g.cuda(), col, nw.cuda(), DV, 1e-6, False, T, gate_act="silu")
        close(got, ref.group_rmsnorm_gate(o, g, col, nw, DV, 1e-6, False, T, gate_act="silu"), dtype, "norm per head times silu of the gate")
    for ta in (torch.float32, T):
        a, c, y = rnd(9, 40, seed=7).to(ta), rnd(9, 40, seed=8), rnd(9, 40, seed=9)
        yd = y.clone().cuda()
        ref.weighted_pair(a, c, 1.3, 0.7, y)
        K.weighted_pair(a.cuda(), c.cuda(), 1.3, 0.7, yd)
        close(yd, y, "float32", "weighted pair")
    lg = rnd(5, 77, seed=10, scale=20.0)
    close(K.softcap(lg.clone().cuda(), 11.0), ref.softcap(lg, 11.0), "float32", "softcap")
    assert float(K.softcap(lg.clone().cuda(), 11.0).abs().max()) <= 11.0
    for M, I, Kd in ((5, 96, 64), (300, 96, 64), (1100, 264, 96)):
        x, w = rnd(M, Kd, seed=11).to(T), rnd(2 * I, Kd, seed=12, scale=0.3).to(T)
        close(K.gate_up_act(x.cuda(), w.cuda(), T, activation="gelu_tanh"), ref.gate_up_act(x, w, T, activation="gelu_tanh"), dtype, f"gelu unit, {M} rows")
    K.check_device_errors()


def test_router_takes_the_largest_corrected_scores_and_weighs_by_the_plain_ones(K):
    ref = TorchKernels()
    for total, top, N in ((10, 2, 33), (3, 3, 5), (70, 5, 200), (512, 8, 9), (4, 1, 1)):
        lg, corr = rnd(N, total, seed=total, scale=2.0), rnd(total, seed=top, scale=0.1)
        for c in (corr, None):
            ids, w = K.moe_route(lg.cuda(), None if c is None else c.cuda(), top)
            ids2, w2 = ref.moe_route(lg, c, top)
            assert torch.equal(ids.cpu(), ids2), (total, top)
            close(w, w2, "float32", "router weights", f32=2e-6)
            assert torch.allclose(w.sum(-1).cpu(), torch.ones(N), atol=1e-5)
    # a correction that turns the order around is used for the choice and left out of the weights
    lg = torch.tensor([[3.0, 2.0, 1.0, 0.0]])
    ids, w = K.moe_route(lg.cuda(), torch.tensor([-1.0, 0.0, 0.0, 1.0]).cuda(), 2)
    s = torch.softmax(lg[0], 0)
    assert ids.cpu().tolist() == [[3, 1]] and torch.allclose(w.cpu()[0], torch.stack([s[3], s[1]]) / (s[3] + s[1]), atol=1e-6)
    # equal scores: the lower index first
    ids, _ = K.moe_route(torch.zeros(2, 6).cuda(), None, 3)
    assert ids.cpu().tolist() == [[0, 1, 2]] * 2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,Kd,total,top", [(1, 64, 5, 2), (9, 44, 3, 3), (130, 72, 7, 1), (33, 1000, 70, 6), (300, 264, 12, 4), (5, 14000, 9, 2)])
def test_router_from_the_rows(K, dtype, N, Kd, total, top):
    """The product and the choice in one kernel (few rows, float32) or as product + choice (prompt portions in bfloat16): the same
    experts as the torch statement wherever its scores are not nearly equal, and the weights of those."""
    ref, T = TorchKernels(), TD[dtype]
    h, w = rnd(N, Kd, seed=1).to(T), (rnd(total, Kd, seed=2) / Kd ** 0.5 * 3).to(T)
    corr = rnd(total, seed=3) * 0.05
    ids, wt = K.moe_router(h.cuda(), w.cuda(), corr.cuda(), top)
    ids2, wt2 = ref.moe_router(h, w, corr, top)
    s = torch.softmax(h.double() @ w.double().T, -1) + corr.double()
    order = torch.sort(s, -1, descending=True).values
    sure = torch.ones(N, dtype=torch.bool) if top == total else (order[:, top - 1] - order[:, top]) > 1e-3
    if top > 1:
        sure &= (order[:, :top - 1] - order[:, 1:top]).min(-1).values > 1e-3   # (the order among the chosen)
    assert bool(sure.any())
    assert torch.equal(ids.cpu()[sure], ids2[sure])
    assert float((wt.cpu()[sure] - wt2[sure]).abs().max()) < (1e-5 if dtype == "float32" else 2e-3)
    one = K.moe_router(h[N - 1:].cuda(), w.cuda(), corr.cuda(), top)
    if dtype == "float32":
        assert torch.equal(one[0], ids[N - 1:]) and torch.equal(one[1], wt[N - 1:]), "a token's choice does not depend on the batch"
    K.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,E,ident,top,Kd,F", [(7, 8, 2, 2, 256, 96), (70, 3, 0, 2, 40, 24), (200, 5, 3, 4, 64, 36), (1, 4, 1, 1, 16, 8), (700, 6, 1, 3, 128, 72),
                                                (300, 2, 4, 5, 48, 16), (1500, 16, 0, 2, 264, 200), (400, 3, 1, 2, 40, 20), (130, 2, 0, 2, 72, 136)])
def test_routed_experts(K, dtype, N, E, ident, top, Kd, F):
    ref, T = TorchKernels(), TD[dtype]
    h = rnd(N, Kd, seed=1).to(T)
    wg, wd = (rnd(E, 2 * F, Kd, seed=2) / Kd ** 0.5).to(T), (rnd(E, Kd, F, seed=3) / F ** 0.5).to(T)
    ids, w = ref.moe_route(rnd(N, E + ident, seed=4), None, top)
    y = rnd(N, Kd, seed=5)
    yd = y.clone().cuda()
    ref.moe_experts(h, ids, w, wg, wd, y)
    K.moe_experts(h.cuda(), ids.cuda(), w.cuda(), wg.cuda(), wd.cuda(), yd)
    close(yd, y, dtype, "routed experts")
    K.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_routed_experts_when_one_expert_takes_all_and_others_none(K, dtype):
    """All tokens on one expert (many tiles of one matrix, the others with no row), only identity experts (no product at all), and
    a token's result not depending on what else is in the batch."""
    ref, T = TorchKernels(), TD[dtype]
    N, E, Kd, F = 333, 5, 64, 40
    h = rnd(N, Kd, seed=1).to(T)
    wg, wd = (rnd(E, 2 * F, Kd, seed=2) / 8).to(T), (rnd(E, Kd, F, seed=3) / 6).to(T)
    for pick in ([3, 6], [5, 6], [4, 0]):                                      # ids 5 and 6 are identity experts
        ids = torch.tensor([pick] * N, dtype=torch.int32)
        w = torch.tensor([[0.75, 0.25]] * N)
        y = torch.zeros(N, Kd)
        yd = y.clone().cuda()
        ref.moe_experts(h, ids, w, wg, wd, y)
        K.moe_experts(h.cuda(), ids.cuda(), w.cuda(), wg.cuda(), wd.cuda(), yd)
        close(yd, y, dtype, f"experts {pick}")
        if pick == [5, 6]:
            close(yd, h.float(), dtype, "two identity experts return the input")
    ids, w = ref.moe_route(rnd(N, E + 2, seed=4), None, 3)
    yd = torch.zeros(N, Kd).cuda()
    K.moe_experts(h.cuda(), ids.cuda(), w.cuda(), wg.cuda(), wd.cuda(), yd)
    for rows in (slice(0, 1), slice(100, 103), slice(332, 333)):
        alone = torch.zeros(rows.stop - rows.start, Kd).cuda()
        K.moe_experts(h[rows].cuda(), ids[rows].cuda(), w[rows].cuda(), wg.cuda(), wd.cuda(), alone)
        if dtype == "float32":
            assert torch.equal(alone, yd[rows]), "a token's experts do not depend on the batch"
        else:
            close(alone, yd[rows], dtype, "a token's experts beside others and alone")
    K.check_device_errors()


# ---------------------------------------------------------------------------------------------------------------------
# the engine

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CASES))
def test_engine_whole_and_cut(cases, name, dtype):
    check_whole_and_cut(cases[(name, dtype)], name, dtype, None, "cuda:0")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CASES))
def test_engine_mixed_batches_on_reused_pages_and_slots(cases, name, dtype):
    check_mixed(cases[(name, dtype)], name, dtype, None, "cuda:0")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CASES))
def test_engine_long_decoding(cases, name, dtype):
    check_long_decoding(cases[(name, dtype)], name, dtype, None, "cuda:0")


@pytest.mark.parametrize("name", sorted(CASES))
def test_float32_does_not_depend_on_how_the_work_is_cut(cases, name):
    """In float32 the recurrences walk their rows in one order, the products, norms and experts treat a row by itself and the
    attention cuts its keys at fixed places: the same bits whole, in portions, and one by one."""
    folder, cfg, tensors, prompts, want = cases[(name, "float32")]
    rp = replayer(folder, name, "float32", 192)
    p = prompts["e"]
    T = len(p)
    whole = run_alone(rp, "w", p, [(0, T)])
    for n, sizes in enumerate(([7, 2, 33, 1, 16, 3, 2, 64, 5], [T - 30] + [1] * 30, [2])):
        got = run_alone(rp, f"c{n}", p, cuts_of(T, sizes), 1000 * (n + 1))
        assert torch.equal(got, whole), f"{name}: portions of {sizes[:3]} differ by {float((got - whole).abs().max()):.3g}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_sharp_scores_show_a_wrong_key(tmp_path, name, dtype):
    """A query norm weight eight times larger makes the softmax pick few keys: a key that is lost or read from a wrong page moves
    the logits by far more than rounding does. Prompt and decoding, portions that end on page borders and one off."""
    folder = make_folder(tmp_path, name, dtype, sharp=8.0, seed=5)
    cfg, tensors = load_plain(folder)
    p = prompt(cfg["vocab"], 140, 21)
    ref = plain_logits(cfg, tensors, p)
    rp = replayer(folder, name, dtype, 192)
    for n, sizes in enumerate(([140], [8, 8, 1, 7, 9, 15, 16, 17], [100] + [1] * 40, [15] + [1] * 125)):
        got = run_alone(rp, f"s{n}", p, cuts_of(140, sizes), 1000 * n)
        err = row_errors(got, ref)
        if dtype == "float32":
            assert float(err.max()) <= 1e-4, f"sharp {name} {sizes[:3]}: {float(err.max()):.3g}"
        else:   # the peaked softmax also magnifies the rounding of q and k, and a router's near tie may fall the other way
            sure = err[~close_calls(ref)]
            assert float(err.median()) <= 0.1 and float(sure.max()) <= 0.5, f"sharp {name} {sizes[:3]}: median {float(err.median()):.3g}, worst {float(sure.max()):.3g}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_entry_point(cases, dtype, graphs):
    from llm_infrence_engine_b200.engine import Engine

    folder, cfg, tensors, prompts, want = cases[("A", dtype)]
    eng = Engine(folder, dtype=dtype, max_len=256, max_seqs=4, block_size=8, num_blocks=70, max_num_batched_tokens=48, cuda_graphs=graphs)
    if graphs:
        assert eng.runner.graphs.usable, "every part of the model only launches kernels: its decode steps are captured"
    ps = [prompts["c"], prompts["d"], prompts["f"], prompts["b"], prompts["e"][:50]]
    results = eng.generate(ps, max_new_tokens=24)
    for p, r in zip(ps, results):
        seq = list(p) + r.token_ids
        whole = plain_logits(cfg, tensors, seq)
        ref, sure = whole[len(p) - 1:-1], ~close_calls(whole)[len(p) - 1:-1]
        if dtype == "float32":
            assert r.token_ids == ref.argmax(-1).tolist()
        else:   # in bfloat16 a near tie may fall the other way: the chosen token must be (nearly) the best one, but where a router's
            # choice hung on two nearly equal scores
            chosen = ref.gather(1, torch.tensor(r.token_ids)[:, None])[:, 0]
            short = (ref.max(-1).values - chosen)[sure]
            assert short.numel() == 0 or float(short.max()) <= 0.05 * float(ref.std())
    eng.cache.check_invariants()
    assert all(pool.num_free == pool.capacity for pool in eng.cache.pools)


def test_preemption_recomputes_the_states(cases):
    """A pool too small for all requests: the youngest is preempted and later recomputed from its first token, its state rows
    starting from zero again. Same tokens as with room for all."""
    from llm_infrence_engine_b200.engine import Engine

    folder, cfg, tensors, prompts, want = cases[("B", "float32")]
    ps = [prompts["b"], prompts["c"], prompts["a"][:60], prompts["e"][:70]]
    big = Engine(folder, dtype="float32", max_len=160, max_seqs=4, block_size=16, num_blocks=60, max_num_batched_tokens=64)
    want_tokens = [r.token_ids for r in big.generate(ps, max_new_tokens=40)]
    small = Engine(folder, dtype="float32", max_len=160, max_seqs=4, block_size=16, num_blocks=19, max_num_batched_tokens=64)
    got = [r.token_ids for r in small.generate(ps, max_new_tokens=40)]
    assert small.preemptions > 0 and got == want_tokens
    small.cache.check_invariants()


def test_random_weights_and_the_command_line(tmp_path):
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    (tmp_path / "cfg.json").write_text(json.dumps(CASES["C"][0]))
    out = subprocess.run([sys.executable, "-m", "llm_infrence_engine_b200", "--model", str(tmp_path / "m"), "--random-weights", str(tmp_path / "cfg.json"),
                          "--dtype", "float32", "--prompt-ids", "1 2 3 4 5", "--max-new-tokens", "6", "--max-len", "64", "--max-seqs", "2"],
                         cwd=root, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    tokens = json.loads(out.stdout.strip().splitlines()[0])["token_ids"]
    cfg, tensors = load_plain(tmp_path / "m")
    seq = [1, 2, 3, 4, 5]
    for t in tokens:
        assert t == int(plain_logits(cfg, tensors, seq)[-1].argmax())
        seq.append(t)
