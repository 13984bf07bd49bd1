"""Memilorn on the GPU: every new kernel against its plain torch statement (and, where one exists, against the plain
implementation's function of the mechanism), and the engine (both dtypes) against the plain implementation: whole prompts, decoding
token by token, portions down to two tokens, mixed batches on reused pages and state slots, long decoding, greedy generation
through the entry point, decode steps from CUDA graphs, and weights and inputs made so that a far key, a lost state, a sink left
out, heads that do not talk or a weight on the wrong side of an expert shows in the result."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_memilorn as plain
from memilorn_cases import (CASES, check_long_decoding, check_mixed, check_whole_and_cut, close_calls, cuts_of, judge, load_plain, make_folder, plain_logits,
                            prompt, replayer, row_errors, run_alone, setup_case, sharpen, tapped_alone)
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
    tmp = tmp_path_factory.mktemp("memilorn")
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


def paged(N_ctx, page, nkv, dk, dv, dtype, seed=0):
    """A pool with one request of ``N_ctx`` tokens on shuffled pages; returns pools, block table and the keys/values in order."""
    pages = -(-N_ctx // page)
    perm = (torch.randperm(pages, generator=torch.Generator().manual_seed(seed)) + 1).to(torch.int32)
    k, v = rnd(N_ctx, nkv, dk, seed=seed + 1).to(TD[dtype]), rnd(N_ctx, nkv, dv, seed=seed + 2).to(TD[dtype])
    k_pool, v_pool = torch.zeros(pages + 2, nkv, page, dk, dtype=TD[dtype]), torch.zeros(pages + 2, nkv, page, dv, dtype=TD[dtype])
    for t in range(N_ctx):
        k_pool[perm[t // page], :, t % page] = k[t]
        v_pool[perm[t // page], :, t % page] = v[t]
    table = torch.zeros(3, pages + 1, dtype=torch.int32)
    table[1, :pages] = perm
    return k_pool, v_pool, table, k, v


# ---------------------------------------------------------------------------------------------------------------------
# the matrix memory

def memory_inputs(N, H, D, DV, dtype, seed=0, pad=8):
    """Rows ``[q | k | v | g]`` with ``pad`` unused columns between the sections, the gates' pre-activations, biases and the norm's weight."""
    T = TD[dtype]
    cols = [0, H * D + pad, 2 * (H * D + pad), 2 * (H * D + pad) + H * DV + pad]
    z = rnd(N, cols[3] + H * DV + 3, seed=seed).to(T)
    gates = rnd(N, 2 * H + 2, seed=seed + 1, scale=2.0)
    return z, cols, gates, rnd(H, seed=seed + 2, scale=0.5), rnd(H, seed=seed + 3, scale=0.5) + 1.5, 1.0 + rnd(H * DV, seed=seed + 4, scale=0.1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,DV,cap,lens", [(3, 8, 16, 4.0, [37, 1, 9]), (2, 12, 12, 15.0, [3, 70]), (4, 16, 8, None, [1, 1, 1]), (2, 64, 64, 6.0, [130]),
                                             (1, 128, 40, 3.0, [20, 5]), (3, 10, 6, 8.0, [2, 1]), (1, 200, 24, 10.0, [1, 33]), (5, 32, 31, 2.0, [8, 9])])
def test_matrix_memory(K, dtype, H, D, DV, cap, lens):
    ref = TorchKernels()
    N = sum(lens)
    z, (qc, kc, vc, gc), gates, bi, bf, nw = memory_inputs(N, H, D, DV, dtype, seed=H + D)
    slots = [5, 0, 3][: len(lens)]
    host, dev = ragged(lens, slots)
    S, M = rnd(7, H, DV + 1, D, seed=1, scale=0.3), rnd(7, H, seed=2).abs()
    Sd, Md = S.clone().cuda(), M.clone().cuda()
    num, m = K.mlstm(z.cuda(), qc, kc, vc, gates.cuda(), bi.cuda(), bf.cuda(), cap, H, D, DV, Sd, Md, dev)
    num2, m2 = ref.mlstm(z, qc, kc, vc, gates, bi, bf, cap, H, D, DV, S, M, host)
    scale = max(1.0, float(num2.abs().max()))
    close(num, num2, "float32", "numerators", scale=scale, f32=1e-5)
    close(m, m2, "float32", "running maximum", f32=1e-6)
    close(Sd, S, "float32", "memory after the step", scale=max(1.0, float(S.abs().max())), f32=1e-5)
    close(Md, M, "float32", "maximum after the step", f32=1e-6)
    y = K.mlstm_finish(num, m, z.cuda(), gc, nw.cuda(), 1e-5, TD[dtype])
    close(y, ref.mlstm_finish(num2, m2, z, gc, nw, 1e-5, TD[dtype]), dtype, "normed and gated result", f32=2e-5)


def test_matrix_memory_against_the_cell_written_out_and_whatever_the_cut(K):
    """One head of the kernel against the plain implementation's loop; and the same bits whether the rows come whole, one by one,
    or in portions whose edges fall inside and between the kernel's tiles of eight tokens."""
    H, D, DV, N, cap = 2, 24, 20, 61, 5.0
    z, (qc, kc, vc, gc), gates, bi, bf, nw = memory_inputs(N, H, D, DV, "float32", seed=3)
    i_log = cap * torch.tanh((gates[:, :H] + bi) / cap)
    f_log = torch.nn.functional.logsigmoid(cap * torch.tanh((gates[:, H:2 * H] + bf) / cap))

    def run(cuts):
        S, M = torch.zeros(3, H, DV + 1, D).cuda(), torch.zeros(3, H).cuda()
        outs = []
        for lo, hi in cuts:
            _, dev = ragged([hi - lo], [1])
            num, m = K.mlstm(z[lo:hi].contiguous().cuda(), qc, kc, vc, gates[lo:hi].contiguous().cuda(), bi.cuda(), bf.cuda(), cap, H, D, DV, S, M, dev)
            outs.append(torch.cat([num.flatten(1), m], dim=1))
        return torch.cat(outs)

    whole = run([(0, N)])
    for h in range(H):
        q = z[:, qc + h * D:qc + (h + 1) * D].double() * D ** -0.5
        k, v = z[:, kc + h * D:kc + (h + 1) * D].double(), z[:, vc + h * DV:vc + (h + 1) * DV].double()
        o = plain.matrix_memory_cell(q, k, v, i_log[:, h].double(), f_log[:, h].double())
        num = whole[:, h * (DV + 1):(h + 1) * (DV + 1)].double().cpu()
        m = whole[:, H * (DV + 1) + h].double().cpu()
        got = num[:, :DV] / (torch.maximum(num[:, DV].abs(), torch.exp(-m)) + 1e-6)[:, None]
        assert float((got - o).abs().max()) <= 2e-5 * max(1.0, float(o.abs().max())), f"head {h}"
    for sizes in ([1], [7, 2, 16, 1, 8, 9], [60, 1], [2]):
        assert torch.equal(run(cuts_of(N, sizes)), whole), f"portions of {sizes} give other bits"


def test_matrix_memory_reads_back_a_far_write(K):
    """Token 0 is written with an open input gate; 400 tokens follow whose input gates are shut and whose forget gates are open; the
    last token asks with token 0's key: it gets token 0's value back, through a state that was carried over 40 steps of a slot
    that another request used before."""
    H, D, DV, N = 2, 32, 16, 401
    z = torch.zeros(N, 2 * H * D + 2 * H * DV)
    key = torch.nn.functional.normalize(rnd(H, D, seed=1), dim=-1) * 4.0
    val = rnd(H, DV, seed=2)
    z[0, H * D:2 * H * D] = key.flatten()
    z[0, 2 * H * D:2 * H * D + H * DV] = val.flatten()
    z[1:, H * D:2 * H * D] = rnd(N - 1, H * D, seed=3)
    z[1:, 2 * H * D:2 * H * D + H * DV] = rnd(N - 1, H * DV, seed=4)
    z[:, :H * D] = rnd(N, H * D, seed=5)
    z[N - 1, :H * D] = key.flatten()
    gates = torch.zeros(N, 2 * H)
    gates[:, :H] = -30.0      # input gates shut ...
    gates[0, :H] = 3.0        # ... but for token 0
    gates[:, H:] = 30.0       # forget gates open: ln sigmoid(30) = -1e-13
    zero = torch.zeros(H)
    S, M = rnd(4, H, DV + 1, D, seed=6).cuda(), rnd(4, H, seed=7).abs().cuda()      # what another request left in the slot
    outs = []
    for n, (lo, hi) in enumerate(cuts_of(N, [11] + [10] * 39)):
        _, dev = ragged([hi - lo], [2])
        if n == 0:
            K.zero_fresh_states([S, M], dev.seq_slots, dev.seq_starts_dev, torch.zeros(hi - lo, dtype=torch.int32).cuda())
        num, m = K.mlstm(z[lo:hi].contiguous().cuda(), 0, H * D, 2 * H * D, gates[lo:hi].contiguous().cuda(), zero.cuda(), zero.cuda(), None, H, D, DV, S, M, dev)
        outs.append((num.cpu(), m.cpu()))
    num, m = outs[-1][0][-1], outs[-1][1][-1]
    got = num[:, :DV] / (torch.maximum(num[:, DV].abs(), torch.exp(-m)) + 1e-6)[:, None]
    assert float((got - val).abs().max()) < 1e-3, float((got - val).abs().max())


# ---------------------------------------------------------------------------------------------------------------------
# heads that talk, a sink, a gate per head

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,dk,dv,cap", [(4, 2, 16, 8, 5.0), (6, 2, 64, 32, 0.0), (3, 3, 24, 40, 2.0), (8, 1, 128, 128, 9.0), (5, 5, 20, 12, 1.5), (16, 4, 64, 64, 30.0),
                                              (2, 1, 48, 32, 0.0)])
def test_attention_whose_heads_talk(K, dtype, nq, nkv, dk, dv, cap):
    """Positions spread over a request of 700 tokens (the first ones, both sides of every slice's and page's border, the last), as a
    prompt portion and as single tokens, with and without sink and gate."""
    ctx_len, page = 700, 16
    k_pool, v_pool, table, _, _ = paged(ctx_len, page, nkv, dk, dv, dtype, 3)
    pos = torch.tensor([0, 1, 2, 15, 16, 17, 255, 256, 257, 300, 511, 512, 513, 640, 698, 699] + list(range(600, 690, 7)), dtype=torch.int32).sort().values
    N = pos.shape[0]
    q = rnd(N, nq * dk + 8, seed=5, scale=0.5).to(TD[dtype])
    gate = rnd(N, nq + 3, seed=6, scale=2.0).to(TD[dtype])
    seq = torch.ones(N, dtype=torch.int32)
    talk = torch.eye(nq) + rnd(nq, nq, seed=7, scale=0.4)
    sink = rnd(nq, seed=8) + 1.0
    for what, kw in {"talk": {}, "talk, sink, gate": dict(sink=sink, gate=gate, gate_col=3, gate_per_head=True), "talk and sink": dict(sink=sink)}.items():
        want = TorchKernels().attention_ext(q, 8, nq, nkv, dk, dv, k_pool, v_pool, table, seq, pos, page, 0.3, 0, ctx_len, softcap=cap, talk=talk, **kw)
        dkw = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in kw.items()}
        for how in ("portion", "single tokens"):
            if how == "portion":
                batch = SimpleNamespace(seq_lens=[N], seq_starts_dev=torch.tensor([0, N], dtype=torch.int32).cuda(), max_seq_len=N, _tables={})
            else:
                batch = SimpleNamespace(seq_lens=[1] * N, seq_starts_dev=torch.arange(N + 1, dtype=torch.int32).cuda(), max_seq_len=1, _tables={})
            got = K.attention_ext(q.cuda(), 8, nq, nkv, dk, dv, k_pool.cuda(), v_pool.cuda(), table.cuda(), seq.cuda(), pos.cuda(), page, 0.3, 0, ctx_len,
                                  batch=batch, softcap=cap, talk=talk.cuda(), **dkw)
            close(got, want, dtype, f"attention_ext {what} ({how})", scale=8.0 if dtype == "float32" else None)
            if how == "portion" and dtype == "bfloat16":   # the tensor-core form took it where the sizes allow: the other form agrees
                K.use_mma_attention_talk = False
                try:
                    other = K.attention_ext(q.cuda(), 8, nq, nkv, dk, dv, k_pool.cuda(), v_pool.cuda(), table.cuda(), seq.cuda(), pos.cuda(), page, 0.3, 0,
                                            ctx_len, batch=batch, softcap=cap, talk=talk.cuda(), **dkw)
                finally:
                    K.use_mma_attention_talk = True
                close(other, want, dtype, f"attention_ext {what} (portion, CUDA cores)")
    fits = K.lib.llmie_attention_talk_mma_fits(nq, nkv, dk, dv)
    assert (fits > 0) == ((nq, nkv, dk, dv) in {(8, 1, 128, 128), (16, 4, 64, 64), (2, 1, 48, 32)}) and fits in (0, 16 * nkv // nq)
    K.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_key_stands_out_through_another_heads_scores(K, dtype):
    """Head 0's own query matches nothing, head 1's query matches one key far back (or at a page's or a slice's border): with a mixing
    matrix that lets head 0 listen to head 1, head 0 returns that key's value; with the identity it does not. The sink, made as
    heavy as the match, takes half of the weight away, once."""
    nq, nkv, dk, dv, ctx_len, page = 2, 1, 32, 16, 1100, 16
    k_pool, v_pool, table, k, v = paged(ctx_len, page, nkv, dk, dv, dtype, 9)
    unit = torch.zeros(dk)
    unit[5] = 1.0
    for key in (3, 255, 256, 1023, 1024, 1087, 1088, 1099):
        kp = k_pool.clone()
        kp[table[1, key // page], 0, key % page] = (unit * 8.0).to(TD[dtype])
        q = torch.zeros(1, nq * dk)
        q[0, dk:] = unit * 8.0                                   # head 1 asks for the key; head 0 asks for nothing
        q = q.to(TD[dtype])
        args = (8 * 0 + 0, nq, nkv, dk, dv, kp.cuda(), v_pool.cuda(), table.cuda(), torch.ones(1, dtype=torch.int32).cuda(), torch.tensor([ctx_len - 1], dtype=torch.int32).cuda(), page, 1.0, 0, ctx_len)
        listen = torch.tensor([[1.0, 1.0], [0.0, 1.0]])
        got = K.attention_ext(q.cuda(), *args, talk=listen.cuda()).float().cpu().view(nq, dv)
        target = v[key, 0].float()
        assert float((got[0] - target).abs().max()) < 0.02 and float((got[1] - target).abs().max()) < 0.02, f"key {key}"
        alone = K.attention_ext(q.cuda(), *args, talk=torch.eye(2).cuda()).float().cpu().view(nq, dv)
        assert float((alone[0] - target).abs().max()) > 0.1 and float((alone[1] - target).abs().max()) < 0.02, f"key {key}, heads that do not talk"
        half = K.attention_ext(q.cuda(), *args, talk=listen.cuda(), sink=torch.tensor([64.0, 64.0]).cuda()).float().cpu().view(nq, dv)
        assert float((half[1] - 0.5 * target).abs().max()) < 0.02, f"key {key} beside a sink of the same weight"


# ---------------------------------------------------------------------------------------------------------------------
# routers that score by sigmoid, weights on the experts' inputs, clamped units, the layer scale, the embedding added again

def test_router_scores_by_sigmoid_and_does_not_renormalise(K):
    ref = TorchKernels()
    for total, top, N in ((10, 2, 33), (3, 3, 5), (70, 5, 200), (4, 1, 1)):
        lg = rnd(N, total, seed=total, scale=2.0)
        ids, w = K.moe_route(lg.cuda(), None, top, scoring="sigmoid")
        ids2, w2 = ref.moe_route(lg, None, top, scoring="sigmoid")
        assert torch.equal(ids.cpu(), ids2), (total, top)
        close(w, w2, "float32", "router weights", f32=2e-6)
    ids, w = K.moe_route(torch.tensor([[3.0, -2.0, 1.0, 0.0]]).cuda(), None, 2, scoring="sigmoid")
    assert ids.cpu().tolist() == [[0, 2]] and torch.allclose(w.cpu()[0], torch.sigmoid(torch.tensor([3.0, 1.0])), atol=1e-6)
    for dtype in DTYPES:
        h, wr = rnd(40, 72, seed=1).to(TD[dtype]), (rnd(6, 72, seed=2) / 3).to(TD[dtype])
        ids, w = K.moe_router(h.cuda(), wr.cuda(), None, 2, scoring="sigmoid")
        z = h.double() @ wr.double().T
        order = torch.sort(z, -1, descending=True).values
        sure = ((order[:, 1] - order[:, 2]) > 1e-2) & ((order[:, 0] - order[:, 1]) > 1e-2)
        ids2, w2 = ref.moe_router(h, wr, None, 2, scoring="sigmoid")
        assert torch.equal(ids.cpu()[sure], ids2[sure]) and float((w.cpu()[sure] - w2[sure]).abs().max()) < (1e-5 if dtype == "float32" else 3e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,E,top,Kd,F,limit", [(7, 8, 1, 256, 96, 2.0), (70, 3, 2, 40, 24, 1.0), (200, 5, 3, 64, 36, 0.7), (1, 4, 1, 16, 8, 3.0), (700, 6, 3, 128, 72, 1.5),
                                                (1500, 16, 2, 264, 200, 2.0), (130, 2, 2, 72, 136, 5.0)])
def test_clamped_experts_with_the_weight_on_their_input(K, dtype, N, E, top, Kd, F, limit):
    ref, T = TorchKernels(), TD[dtype]
    h = rnd(N, Kd, seed=1).to(T)
    wg, wd = (rnd(E, 2 * F, Kd, seed=2) / Kd ** 0.5 * 2).to(T), (rnd(E, Kd, F, seed=3) / F ** 0.5).to(T)
    ids, w = ref.moe_route(rnd(N, E, seed=4), None, top, scoring="sigmoid")
    y = rnd(N, Kd, seed=5)
    yd = y.clone().cuda()
    glu = (limit, 1.702, 1.0)
    ref.moe_experts(h, ids, w, wg, wd, y, glu=glu, weight_inputs=True)
    K.moe_experts(h.cuda(), ids.cuda(), w.cuda(), wg.cuda(), wd.cuda(), yd, glu=glu, weight_inputs=True)
    close(yd, y, dtype, "clamped experts, weighted inputs")
    # the weight on the OUTPUT instead is another function (the unit is not linear): the test's inputs tell the two apart
    other = rnd(N, Kd, seed=5)
    ref.moe_experts(h, ids, w, wg, wd, other, glu=glu, weight_inputs=False)
    assert float((other - y).abs().max()) > 0.01
    K.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_layer_scale_is_added_with_the_next_norm_and_the_embedding_once_more(K, dtype):
    T = TD[dtype]
    N, W = 37, 72
    x, y, ls, w = rnd(N, W, seed=1), rnd(N, W, seed=2), 1.0 + rnd(W, seed=3, scale=0.3), 1.0 + rnd(W, seed=4, scale=0.1)
    table, ids = rnd(50, W, seed=5).to(T), torch.randint(0, 50, (N,), generator=torch.Generator().manual_seed(6), dtype=torch.int32)
    want_x = x + y * ls + table[ids.long()].float()
    mu = want_x.mean(-1, keepdim=True)
    want_h = (want_x - mu) / torch.sqrt(((want_x - mu) ** 2).mean(-1, keepdim=True) + 1e-5) * w
    for how in ("with the norm", "flushed", "at chosen rows"):
        xd = x.clone().cuda()
        buf = K.zeros_like_rows(xd)
        buf += y.cuda()
        K._unfresh(buf)
        K.scaled_add(xd, buf, ls.cuda())
        K.embed_add(ids.cuda(), table.cuda(), xd)              # (the scaled result still waits; additions commute)
        if how == "flushed":
            K.flush()
            close(xd, want_x, "float32", "stream after the flush", f32=2e-6)
        rows = torch.tensor([3, 0, 36], dtype=torch.int32) if how == "at chosen rows" else None
        h = K.layernorm(xd, w.cuda(), 1e-5, T, rows.cuda() if rows is not None else None)
        close(h, want_h if rows is None else want_h[rows.long()], dtype, f"norm {how}", f32=1e-5)
        if rows is None:
            close(xd, want_x, "float32", f"stream {how}", f32=2e-6)
        assert float(K.zeros_like_rows(xd).abs().max()) == 0.0, "the buffer is zero again for its next user"


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
    """In float32 the memory walks its rows in one order, the products, norms and experts treat a row by itself and the attention cuts
    its keys at fixed places: the same bits whole, in portions, and one by one."""
    folder, cfg, tensors, prompts, want = cases[(name, "float32")]
    rp = replayer(folder, name, "float32", 192)
    p = prompts["e"]
    T = len(p)
    whole = run_alone(rp, "w", p, [(0, T)])
    for n, sizes in enumerate(([7, 2, 33, 1, 16, 3, 2, 64, 5], [T - 30] + [1] * 30, [2])):
        got = run_alone(rp, f"c{n}", p, cuts_of(T, sizes), 1000 * (n + 1))
        assert torch.equal(got, whole), f"{name}: portions of {sizes[:3]} differ by {float((got - whole).abs().max()):.3g}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CASES))
def test_sharp_weights_show_a_wrong_key_a_lost_state_or_a_sink_left_out(tmp_path, name, dtype):
    """Queries eight times larger, heads that listen to each other, heavy sinks and a memory that forgets slowly: a key that is lost
    or read from a wrong page, a state that is not carried, a sink or a mix that is left out moves the logits by far more than
    rounding does. Prompt and decoding, portions that end on page borders and one off, a request of 600 tokens (several slices)."""
    folder = make_folder(tmp_path, name, dtype, seed=5, tweak=sharpen, tag="_sharp")
    cfg, tensors = load_plain(folder)
    # the oracle itself must feel every sharpened mechanism, or the test shows nothing
    p = prompt(cfg["vocab"], 140, 21)
    ref = plain_logits(cfg, tensors, p)
    for gone in (".sink", ".talk", ".f.b"):
        t2 = {k: v.clone() for k, v in tensors.items()}
        for key in t2:
            if key.endswith(gone):
                t2[key] = torch.eye(t2[key].shape[0]) if gone == ".talk" else t2[key] - (5.0 if gone == ".sink" else 4.0)
        if any(key.endswith(gone) for key in t2):
            assert float(row_errors(plain_logits(cfg, t2, p), ref).median()) > 0.02, f"{name}: the oracle does not feel {gone}"
    rp = replayer(folder, name, dtype, 640)
    # (the peaked softmax also magnifies the rounding of q and k: the bfloat16 bound is wider than for plain weights, and still far
    # below what a lost key, state, sink or mix does, see above)
    limit = 1e-4 if dtype == "float32" else 0.15
    for n, sizes in enumerate(([140], [8, 8, 1, 7, 9, 15, 16, 17], [100] + [1] * 40, [15] + [1] * 125)):
        got, choices = tapped_alone(rp, cfg, f"s{n}", p, cuts_of(140, sizes), 1000 * n)
        judge(got, cfg, tensors, p, choices, dtype, f"sharp {name} {sizes[:3]}", limit=limit, own=ref)
    long = prompt(cfg["vocab"], 600, 22)
    got, choices = tapped_alone(rp, cfg, "long", long, cuts_of(600, [255, 2, 256, 1, 60] + [1] * 30), 9000)
    judge(got, cfg, tensors, long, choices, dtype, f"sharp {name}, 600 tokens", limit=limit)


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
        else:   # in bfloat16 a near tie may fall the other way, between two tokens or between two experts (which then moves the later
            # logits too): most chosen tokens are (nearly) the best ones of the oracle run on the same sequence
            chosen = ref.gather(1, torch.tensor(r.token_ids)[:, None])[:, 0]
            short = ref.max(-1).values - chosen
            assert float((short <= 0.05 * float(ref.std())).float().mean()) >= 0.75, short
    eng.cache.check_invariants()
    assert all(pool.num_free == pool.capacity for pool in eng.cache.pools)


def test_preemption_recomputes_the_states(cases):
    """A pool too small for all requests: the youngest is preempted and later recomputed from its first token, its memory starting
    from zero again. Same tokens as with room for all."""
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
