"""Small Mufotar models and the ways of running them that the CPU and the GPU tests share.

The configurations differ from each other in every size and option: layer orders, layers that run on another layer's weights
(an earlier and a later one), query/key groups of 1, 2 and 3, keys and values of equal and of different sizes, heads turned in
part, in full and not at all, convolutions of 1 to 8 taps, states of 12 to 40, step-size ranks of 1, 3, 5 and 8, routers that
choose 1, 2, 3 and 4 of their outputs with 0 to 3 identity experts, with and without a shared unit, layers with a dense
feed-forward and with none, logits with and without a soft cap. The engine runs them through ``TraceReplayer`` (the step
function, the cache manager, the kernels object it is given); the oracle is ``plain_mufotar.forward`` on whole sequences.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

import plain_mufotar as plain
from luvutar_cases import cuts_of, load_plain, prompt, run_alone, run_mixed  # noqa: F401  (generic helpers)


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def _parallel(left, right, scales):
    heads, kv_heads, dim, vdim, scale, rot = left
    lm = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        lm["rot"] = {"dims": rot[0], "base": rot[1]}
    rm = dict(zip(("inner", "state", "dt_rank", "conv"), right))
    return {"type": "parallel", "mixer": {"left": lm, "right": rm, "left_scale": scales[0], "right_scale": scales[1]}}


def _dense(layer, ff):
    layer = json.loads(json.dumps(layer))
    layer["mlp"] = {"kind": "dense", "ff": ff} if ff else None
    return layer


def _moe(layer, experts, identity, top, ff, shared):
    layer = json.loads(json.dumps(layer))
    layer["mlp"] = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared:
        layer["mlp"]["shared"] = {"ff": shared}
    return layer


def _again(layers, j):
    layer = json.loads(json.dumps(layers[j]))
    layer["weights_of"] = j
    return layer


def _model(vocab, width, eps, softcap, layers, again=()):
    layers = list(layers)
    for j in again:
        layers.append(_again(layers, j))
    cfg = {"architecture": "Mufotar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if softcap:
        cfg["logit_softcap"] = softcap
    return cfg


CASES = {
    # (config, page size). A: both mixers; partly turned heads; three of seven router outputs, two of them identity experts, a shared
    # unit; a layer without feed-forward; two layers run again on earlier weights, in another order; pages of 8
    "A": (_model(83, 48, 1e-5, 12.0, [
        _dense(_delta(4, 2, 16, 24, 3), 64),
        _moe(_parallel((6, 2, 24, 16, 0.2, (16, 1000.0)), (40, 12, 5, 4), (0.7, 1.3)), 5, 2, 3, 24, 40),
        _dense(_delta(3, 3, 8, 40, 4), None),
    ], again=(1, 0)), 8),
    # B: the side-by-side mixer first; one key/value head; fully turned heads of 64; an attention without rotation; one expert of
    # three and no identity expert, no shared unit; no soft cap on the logits; sizes that are no multiples of 32
    "B": (_model(120, 64, 1e-6, None, [
        _moe(_parallel((2, 1, 64, 64, 0.125, (64, 10000.0)), (72, 16, 8, 2), (1.0, 1.0)), 3, 0, 1, 32, None),
        _moe(_delta(2, 1, 32, 16, 2), 4, 1, 2, 16, 24),
        _dense(_parallel((3, 3, 8, 8, 0.35, None), (24, 40, 3, 3), (0.5, 2.0)), 96),
    ], again=(1,)), 16),
}
# C: sizes that take the kernels' slow paths: a width that is no multiple of 8, heads of 20 and 10 entries (no 16-byte pieces), values
# of 12 and 6, a convolution of 8 taps and one of a single tap (no state rows at all), a step-size rank of 1, four of five router
# outputs of which three are identity experts, pages of 4, and a first layer that runs on the weights of a LATER one
_c_layers = [_moe(_delta(3, 1, 10, 6, 8), 2, 3, 4, 12, 20), _dense(_parallel((4, 2, 20, 12, 0.22, (6, 7.0)), (36, 20, 1, 1), (1.1, 0.4)), 52),
             _moe(_delta(3, 1, 10, 6, 8), 2, 3, 4, 12, 20)]
_c_layers[0]["weights_of"] = 2
CASES["C"] = (_model(57, 44, 1e-6, 5.0, _c_layers), 4)

LENS = {"a": 150, "b": 67, "c": 41, "d": 9, "e": 118, "f": 2}

# float32: only the order of summation differs. bfloat16: activations are rounded to 8 bits between the kernels; a wrong key, a
# lost state or a wrong expert moves the logits by 0.3 and more
LIMIT = {"float32": 3e-5, "bfloat16": 1e-1}


def make_folder(tmp: Path, name: str, store: str = "float32", std: float = 0.08, seed: int = 11, sharp: float = 1.0) -> Path:
    """A model folder for case ``name`` with random weights. ``sharp`` multiplies the weight of the queries' norm (the queries are
    normed, so scaling their projection would change nothing), so that the softmax picks few keys and a key that is lost, or
    read from a wrong page, moves the logits by far more than rounding does."""
    from llm_infrence_engine_b200.weights.random_init import random_tensors
    from llm_infrence_engine_b200.weights.safetensors_io import write_safetensors

    cfg, _ = CASES[name]
    t = random_tensors(cfg, seed, std)
    if sharp != 1.0:
        for key in t:
            if key.endswith("left.q.norm"):
                t[key] = t[key] * sharp
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[store]
    folder = Path(tmp) / f"mufotar_{name}_{store}_{sharp}"
    folder.mkdir(parents=True, exist_ok=True)
    write_safetensors(folder / "model.safetensors", {k: v.to(dtype).contiguous() for k, v in t.items()})
    (folder / "config.json").write_text(json.dumps(cfg))
    return folder


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


def judge(got, want, dtype, what, limit=None):
    """float32: every row within the limit. bfloat16: a router's choice between two nearly equal scores may fall the other way
    than in the 64-bit oracle, which moves that token's logits (and, through the states, later ones) by more than rounding does:
    so nearly all rows are within the limit, and none is far off but where the oracle itself saw such a close call."""
    err = row_errors(got, want)
    close = close_calls(want)
    limit = limit or LIMIT[dtype]
    if dtype == "float32":
        assert float(err.max()) <= limit, f"{what}: {float(err.max()):.3g}"
    else:
        sure = err[~close]
        over, far = int((sure > limit).sum()), float(sure.max()) if sure.numel() else 0.0
        assert over <= max(2, err.numel() // 20) and far <= 4 * limit, f"{what}: {over} of {err.numel()} rows over, worst {far:.3g} ({int(close.sum())} close calls left out)"


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
            got = run_alone(rp, f"{k}{n}", p, cuts, n)
            n += len(cuts)
            judge(got, want[k], dtype, f"{name} {dtype} request {k} ({T} tokens) {what}")
            rp.cache.check_invariants()
    assert rp.cache.num_free_slots() == 4 and all(p.num_free == p.capacity for p in rp.cache.pools)


def check_mixed(case, name, dtype, kernels, device, seeds=(0, 1)):
    """Batches of unequal requests on a pool that holds only the live ones (pages and state slots are used again): every
    request as if it ran alone."""
    folder, cfg, tensors, prompts, want = case
    for seed in seeds:
        lens = sorted((len(p) for p in prompts.values()), reverse=True)
        rp = replayer(folder, name, dtype, sum(-(-n // 64) * 64 for n in lens[:4]), kernels, device)
        got = run_mixed(rp, prompts, seed)
        for k in prompts:
            judge(got[k], want[k], dtype, f"{name} {dtype} mixed (seed {seed}) request {k}")
        assert rp.cache.num_free_slots() == 4 and all(p.num_free == p.capacity for p in rp.cache.pools)


def check_long_decoding(case, name, dtype, kernels, device, total=300):
    """A short prompt, then hundreds of tokens one by one: the states run on, the keys grow over many pages."""
    folder, cfg, tensors, prompts, want = case
    p = prompt(cfg["vocab"], total, 99)
    ref = plain_logits(cfg, tensors, p)
    rp = replayer(folder, name, dtype, 320, kernels, device)
    got = run_alone(rp, "long", p, cuts_of(total, [3] + [1] * total))
    judge(got, ref, dtype, f"{name} {dtype} long decoding")
    judge(got[:4], ref[:4], dtype, f"{name} {dtype} first tokens")
