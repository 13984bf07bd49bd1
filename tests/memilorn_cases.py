"""Small Memilorn models and the ways of running them that the CPU and the GPU tests share.

The configurations differ from each other in every size and option: layer orders; loops of 3, 2 and no passes that start at the
first layer or later and are followed by further layers or not; query heads per key/value head of 3, 1 and 2; keys and values of
equal and of different sizes; heads turned in part, in full and not at all; scores with and without a soft cap; gates of the memory
with and without a cap; routers that choose 2, 1 and 3 of their experts, with and without a shared unit; layers without a
feed-forward. The engine runs them through ``TraceReplayer`` (the step function, the cache manager, the kernels object it is given);
the oracle is ``plain_memilorn.forward`` on whole sequences.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

import plain_memilorn as plain
from luvutar_cases import cuts_of, load_plain, prompt, run_alone, run_mixed  # noqa: F401  (generic helpers)


def _memory(heads, dim, vdim, cap):
    m = {"heads": heads, "dim": dim, "vdim": vdim}
    if cap:
        m["gate_cap"] = cap
    return {"type": "mlstm", "mixer": m}


def _latent(heads, dim, vdim, kv_rank, scale):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}}


def _attention(heads, kv_heads, dim, vdim, scale, rot, softcap):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if softcap:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m}


def _moe(layer, experts, top, ff, limit, shared=None):
    layer = json.loads(json.dumps(layer))
    if experts is None:
        layer["mlp"] = None
        return layer
    layer["mlp"] = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        layer["mlp"]["shared"] = {"ff": shared[0], "limit": shared[1]}
    return layer


def _model(vocab, width, eps, layers, loop=None):
    cfg = {"architecture": "Memilorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": list(layers)}
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


CASES = {
    # (config, page size). A: all three mixers; three query heads per key/value head; partly turned heads; layers 1 and 2 run three
    # times and a layer follows the loop; two of five experts and a shared unit; pages of 8
    "A": (_model(83, 48, 1e-5, [
        _moe(_attention(6, 2, 16, 8, 0.3, (8, 100.0), 5.0), 5, 2, 24, 1.5, (40, 2.5)),
        _moe(_memory(3, 8, 16, 4.0), 5, 2, 24, 1.5, (40, 2.5)),
        _moe(_latent(4, 8, 12, 16, 0.4), 4, 3, 16, 3.0),
        _moe(_memory(2, 12, 12, 15.0), None, None, None, None),
    ], loop=(1, 3, 3)), 8),
    # B: no loop at all; latent attention first; every query head its own key/value head, heads turned in full, no soft cap; a memory
    # whose gates have no cap; one expert of three without a shared unit; a layer without feed-forward in the middle; pages of 16
    "B": (_model(120, 64, 1e-6, [
        _moe(_latent(2, 16, 16, 24, 0.25), 3, 1, 32, 2.0),
        _moe(_attention(3, 3, 32, 32, 0.18, (32, 10000.0), None), None, None, None, None),
        _moe(_memory(4, 16, 8, None), 6, 3, 16, 1.0, (24, 4.0)),
    ]), 16),
    # C: sizes that take the kernels' slow paths: a width that is no multiple of 8, heads of 20 and 10 entries (no 16-byte pieces), values
    # of 12 and 6, a latent of 20, an attention without rotation; the loop starts at the first layer and runs twice; pages of 4
    "C": (_model(57, 44, 1e-6, [
        _moe(_memory(3, 10, 6, 8.0), 2, 2, 12, 2.0, (20, 2.0)),
        _moe(_attention(4, 2, 20, 12, 0.22, None, 9.0), 3, 1, 20, 1.2),
        _moe(_latent(3, 10, 6, 20, 0.3), 3, 2, 12, 2.0, (12, 1.0)),
    ], loop=(0, 2, 2)), 4),
}

LENS = {"a": 150, "b": 67, "c": 41, "d": 9, "e": 118, "f": 2}

# float32: only the order of summation differs. bfloat16: activations are rounded to 8 bits between the kernels; a wrong key, a
# lost state, a sink left out or a wrong expert moves the logits by 0.3 and more
LIMIT = {"float32": 3e-5, "bfloat16": 1e-1}


def make_folder(tmp: Path, name: str, store: str = "float32", std: float = 0.08, seed: int = 11, tweak=None, tag: str = "") -> Path:
    """A model folder for case ``name`` with random weights. ``tweak(tensors)`` may change them in place before they are written (a
    test that wants peaked scores, a heavy sink, heads that really talk or a memory that forgets slowly says so there)."""
    from llm_infrence_engine_b200.weights.random_init import random_tensors
    from llm_infrence_engine_b200.weights.safetensors_io import write_safetensors

    cfg, _ = CASES[name]
    t = random_tensors(cfg, seed, std)
    if tweak is not None:
        tweak(t)
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[store]
    folder = Path(tmp) / f"memilorn_{name}_{store}{tag}"
    folder.mkdir(parents=True, exist_ok=True)
    write_safetensors(folder / "model.safetensors", {k: v.to(dtype).contiguous() for k, v in t.items()})
    (folder / "config.json").write_text(json.dumps(cfg))
    return folder


def sharpen(t: dict) -> None:
    """Weights under which a fault shows: queries eight times larger (the softmax picks few keys, so a lost or misplaced key moves
    the logits), heads that take a third of their scores from their neighbours, sinks as heavy as the best key, a memory that
    forgets slowly (forget gates near one) and takes in strongly."""
    g = torch.Generator().manual_seed(7)
    for key in list(t):
        if key.endswith(".mix.q") and (key[:-1] + "dkv" in t or key[:-1] + "talk" in t):
            t[key] = t[key] * 8.0
        if key.endswith(".talk"):
            t[key] = t[key] + torch.randn(t[key].shape, generator=g) * 0.35
        if key.endswith(".sink"):
            t[key] = t[key] + 5.0
        if key.endswith(".f.b"):
            t[key] = t[key] + 4.0


def replayer(folder, name, dtype, max_tokens, kernels=None, device="cuda:0", **kw):
    from llm_infrence_engine_b200.engine import TraceReplayer

    return TraceReplayer(str(folder), dtype, max_tokens, device=device, kernels=kernels, block_size=CASES[name][1], **kw)


def plain_logits(cfg, tensors, tokens):
    """The oracle's logits; ``close_calls`` of the result marks the tokens at which some router's choice hung on two nearly equal
    scores (a slice of the result loses the mark and is judged without it)."""
    close = []
    logits = plain.forward(cfg, tensors, tokens, torch.float64, close_out=close)
    logits.close_calls = torch.stack(close).any(0) if close else torch.zeros(len(tokens), dtype=torch.bool)
    return logits


def close_calls(logits: torch.Tensor) -> torch.Tensor:
    return getattr(logits, "close_calls", torch.zeros(logits.shape[0], dtype=torch.bool))


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """The difference of every row of logits (its mean taken off, root mean square over the vocabulary), in units of the logits' spread."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / want.double().std()


class RouterTap:
    """Listens to the routers of a kernels object: what every call chose, in the order of the calls (a step calls once per run of a
    feed-forward, in running order, with the step's rows). With it the oracle can be made to take the SAME experts as the engine,
    so that in bfloat16 a choice that hung on rounding does not count as a difference; that the engine's choice was a sound one is
    judged separately (``judge_choices``)."""

    def __init__(self, kernels):
        self.K, self.calls = kernels, []
        inner = kernels.moe_router

        def listening(h, w_router, correction, top, scoring="softmax"):
            ids, weights = inner(h, w_router, correction, top, scoring)
            self.calls.append(ids.detach().cpu().long())
            return ids, weights

        kernels.moe_router = listening

    def close(self):
        del self.K.moe_router     # (the instance's attribute; the class's method is back)

    def choices(self, runs: int, rows_of: list, order: list) -> dict:
        """From the calls of a sequence of steps: per request, a list over the feed-forward runs of ``[T, top]``. ``rows_of[s]`` lists
        ``(request, rows)`` of step s in batch order."""
        out = {r: [[] for _ in range(runs)] for r in order}
        assert len(self.calls) == runs * len(rows_of), f"{len(self.calls)} router calls for {len(rows_of)} steps of {runs} runs"
        for s, step in enumerate(rows_of):
            for j in range(runs):
                ids, o = self.calls[s * runs + j], 0
                for rid, n in step:
                    out[rid][j].append(ids[o:o + n])
                    o += n
        return {r: [torch.cat(c) for c in per] for r, per in out.items()}


def moe_runs(cfg) -> int:
    return sum(1 for i, _ in plain.running_order(cfg) if cfg["layers"][i].get("mlp"))


def tapped_alone(rp, cfg, rid, tokens, cuts, step0=0):
    """``run_alone`` with the routers' choices: (logits [T, vocab], per feed-forward run [T, top])."""
    tap = RouterTap(rp.runner.K)
    try:
        got = run_alone(rp, rid, tokens, cuts, step0)
    finally:
        tap.close()
    return got, tap.choices(moe_runs(cfg), [[(rid, hi - lo)] for lo, hi in cuts], [rid])[rid]


def judge(got, cfg, tensors, tokens, choices, dtype, what, limit=None, own=None):
    """The engine's logits against the oracle's. float32: every row within the limit, the oracle taking its own experts (one row in
    fifty may be ten times off: a position where a head's normaliser n . q nearly cancels is ill-conditioned in 32-bit, for the
    oracle's own formulas run in 32-bit too). bfloat16: the oracle takes the experts the engine took, and nearly all rows are within
    the limit and none far off; and the engine's experts are the router's own choice but where that hung on less than a quarter of
    the router's largest output (measured: up to 0.12, at tokens where the memory's normaliser nearly cancels and rounding to 8 bits
    moves the stream by several percent; an expert taken at random lies a whole largest output below)."""
    limit = limit or LIMIT[dtype]
    if dtype == "float32":
        want = own if own is not None else plain.forward(cfg, tensors, tokens, torch.float64)
        err = row_errors(got, want)
        over = int((err > limit).sum())
        assert over <= err.numel() // 50 + (err.numel() >= 20) and float(err.max()) <= 10 * limit, f"{what}: {over} rows over, worst {float(err.max()):.3g}"
        return
    regret = []
    want = plain.forward(cfg, tensors, tokens, torch.float64, forced=choices, regret_out=regret)
    err = row_errors(got, want)
    over, far = int((err > limit).sum()), float(err.max())
    assert over <= max(2, err.numel() // 20) and far <= 4 * limit, f"{what}: {over} of {err.numel()} rows over, worst {far:.3g}"
    if regret:
        worst = float(torch.stack(regret).max())
        assert worst <= 0.25, f"{what}: a router took an expert whose output lies {worst:.3g} of the largest below its own choice"


def setup_case(tmp, name, dtype, **kw):
    folder = make_folder(tmp, name, dtype, **kw)
    cfg, tensors = load_plain(folder)
    prompts = {k: prompt(cfg["vocab"], n, 3 + i) for i, (k, n) in enumerate(LENS.items())}
    want = {k: plain_logits(cfg, tensors, p) for k, p in prompts.items()}
    return folder, cfg, tensors, prompts, want


# ---------------------------------------------------------------------------------------------------------------------
# The checks themselves: each takes the kernels object and the device, so the same statements run on the CPU (torch
# stand-in kernels: the host side of the engine) and on the GPU (the package's kernels).

def check_whole_and_cut(case, name, dtype, kernels, device, only=None):
    """Whole prompts; the last tokens one by one; portions of several sizes down to two tokens and one."""
    folder, cfg, tensors, prompts, want = case
    rp = replayer(folder, name, dtype, 192, kernels, device)
    n = 0
    for k, p in prompts.items():
        if only and k not in only:
            continue
        T = len(p)
        ways = {"whole": [(0, T)], "tail one by one": cuts_of(T, [max(1, T - 40)] + [1] * 40),
                "portions": cuts_of(T, [7, 2, 33, 1, 16, 3, 2, 64, 5]), "pairs": cuts_of(T, [2])}
        for what, cuts in ways.items():
            if what == "pairs" and T > 70:
                continue
            got, choices = tapped_alone(rp, cfg, f"{k}{n}", p, cuts, n)
            n += len(cuts)
            judge(got, cfg, tensors, p, choices, dtype, f"{name} {dtype} request {k} ({T} tokens) {what}", own=want[k])
            rp.cache.check_invariants()
    assert rp.cache.num_free_slots() == 4 and all(p.num_free == p.capacity for p in rp.cache.pools)


def check_mixed(case, name, dtype, kernels, device, seeds=(0, 1)):
    """Batches of unequal requests on a pool that holds only the live ones (pages and state slots are used again): every
    request as if it ran alone."""
    from luvutar_cases import mixed_schedule

    folder, cfg, tensors, prompts, want = case
    lens = {k: len(v) for k, v in prompts.items()}
    for seed in seeds:
        longest = sorted(lens.values(), reverse=True)
        rp = replayer(folder, name, dtype, sum(-(-n // 64) * 64 for n in longest[:4]), kernels, device)
        tap = RouterTap(rp.runner.K)
        got, rows_of = {k: [] for k in prompts}, []
        try:
            for n, step in enumerate(mixed_schedule(lens, seed)):
                entries = [{"id": rid, "tokens": prompts[rid][lo:hi], "want": list(range(hi - lo))} for rid, lo, hi in step]
                out = rp.step({"step": n, "entries": entries, "end": [rid for rid, lo, hi in step if hi == lens[rid]]})
                rp.cache.check_invariants()
                rows_of.append([(rid, hi - lo) for rid, lo, hi in step])
                o = 0
                for rid, lo, hi in step:
                    got[rid].append(out[o:o + hi - lo])
                    o += hi - lo
        finally:
            tap.close()
        choices = tap.choices(moe_runs(cfg), rows_of, list(prompts))
        for k in prompts:
            judge(torch.cat(got[k]), cfg, tensors, prompts[k], choices[k], dtype, f"{name} {dtype} mixed (seed {seed}) request {k}", own=want[k])
        assert rp.cache.num_free_slots() == 4 and all(p.num_free == p.capacity for p in rp.cache.pools)


def check_long_decoding(case, name, dtype, kernels, device, total=300):
    """A short prompt, then hundreds of tokens one by one: the memory runs on, the keys grow over many pages."""
    folder, cfg, tensors, prompts, want = case
    p = prompt(cfg["vocab"], total, 99)
    rp = replayer(folder, name, dtype, 320, kernels, device)
    got, choices = tapped_alone(rp, cfg, "long", p, cuts_of(total, [3] + [1] * total))
    judge(got, cfg, tensors, p, choices, dtype, f"{name} {dtype} long decoding")
    judge(got[:4], cfg, tensors, p[:4], [c[:4] for c in choices], dtype, f"{name} {dtype} first tokens")
