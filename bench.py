"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of Qwen2.5-0.5B (24 layers, hidden 896, 14 query / 2 key-value
heads of 64, intermediate 4864, vocabulary 151936, tied head) with random weights in bfloat16, a
batch of 8 requests and a context of 8192 tokens. A "step" is one decode step of the whole batch.

``value``     decoded tokens per second of the step function alone: W warm-up steps, then K steps
              between two CUDA events on the launching stream with a synchronize on both sides.
              The requests' cache pages hold synthetic keys and values (a step's cost does not
              depend on them); weights plus cache are far larger than L2, so nothing is flushed.
``e2e``       the same through ``Engine.step()``: requests are added as token lists on the host,
              their prompts are prefilled by the engine, and every timed step copies its inputs
              from pinned host memory and reads sampled tokens back (the engine runs pipelined: a
              step is launched before the tokens of the step before it have been read).
``prefill``   one prompt of 2,048 tokens in one step (device time between two events, median of five runs after three
              warm-up runs; a step shape that recurs is replayed from a CUDA graph, as in serving);
              ``frac`` = flops / time / bfloat16 peak.
``roofline``  bytes a decode step must read (every weight once + the live requests' cache) / its time.
``points``    decode tokens per second at batch 1 and 64, same method as ``value``.

``--workload serving | luvutar | zepalorn | mufotar | memilorn`` measure other things (a stream of requests through the engine; the other architectures
beside Qwen2 of equal size, Mufotar beside Zepalorn, with ``--kernels`` also kernel by kernel) and print lines of their own; the default line is
unchanged by them.

Peaks come from MEASURED_PEAKS.json beside this file when it exists, else 6.65 TB/s and 1.59 PFLOP/s.
More than one GPU is outside this engine: ``--gpus N`` with N > 1 prints one line and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

MODEL = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": 151936, "hidden_size": 896,
    "intermediate_size": 4864, "num_hidden_layers": 24, "num_attention_heads": 14, "num_key_value_heads": 2,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": True, "max_position_embeddings": 32768,
    "use_sliding_window": False, "hidden_act": "silu",
}
CONTEXT = 8192
PREFILL_TOKENS = 2048
BLOCK = 16

# Other layer sizes of the same architecture (``--shape``): what changes against MODEL, and the context length they are quoted at.
SHAPES = {
    "0.5b": ("Qwen2.5-0.5B shape", {}, 8192),
    "1.5b": ("Qwen2.5-1.5B shape", {"hidden_size": 1536, "intermediate_size": 8960, "num_hidden_layers": 28, "num_attention_heads": 12,
                                    "num_key_value_heads": 2}, 8192),
    "7b": ("Qwen2.5-7B shape", {"vocab_size": 152064, "hidden_size": 3584, "intermediate_size": 18944, "num_hidden_layers": 28,
                                "num_attention_heads": 28, "num_key_value_heads": 4, "tie_word_embeddings": False}, 16384),
}


def peaks() -> dict:
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            d = json.loads(p.read_text())
            if d.get("hbm_gbs"):
                out["hbm_gbs"] = float(d["hbm_gbs"])
            if d.get("bf16_tflops"):
                out["bf16_tflops"] = float(d["bf16_tflops"])
            if d.get("bf16_tflops_sustained"):
                out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
            out["source"] = "measured"
        except (ValueError, OSError):
            pass
    return out


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of GPU 0 every 100 ms while running."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons}


def flops_prefill(T: int) -> float:
    m = MODEL
    d = m["hidden_size"] // m["num_attention_heads"]
    per_layer = (m["hidden_size"] * (m["num_attention_heads"] + 2 * m["num_key_value_heads"]) * d
                 + m["num_attention_heads"] * d * m["hidden_size"] + 3 * m["hidden_size"] * m["intermediate_size"])
    linear = 2.0 * T * per_layer * m["num_hidden_layers"]
    attn = m["num_hidden_layers"] * 4.0 * m["num_attention_heads"] * d * (T * (T + 1) / 2)
    head = 2.0 * m["hidden_size"] * m["vocab_size"]
    return linear + attn + head


REF_DIR = ROOT / "baseline" / "_ref"


def _reference_model(folder: Path, torch):
    """The reference's own model from a model folder, built the way its loader does (src/miniserve/loader.py:36-48:
    ``ModelConfig.from_json``, ``Qwen2`` on the meta device, ``load_state_dict(assign=True)``, the tie re-established), without the
    tokenizer and the download that ``load_model`` adds."""
    from miniserve.model import ModelConfig, Qwen2
    from safetensors.torch import load_file

    cfg = ModelConfig.from_json(folder / "config.json")
    with torch.device("meta"):
        model = Qwen2(cfg)
    state = {}
    for f in sorted(folder.glob("*.safetensors")):
        state.update(load_file(f))
    model.load_state_dict(state, strict=False, assign=True)
    if cfg.tie_word_embeddings:
        model.lm_head.weight = model.model.embed_tokens.weight
    return model.to(device="cuda:0", dtype=torch.bfloat16).eval()


def _reference_decode(model, torch, kind: str, batch: int, steps: int, warmup: int) -> dict:
    """``steps`` decode steps of ``batch`` requests whose contexts reach CONTEXT, through the reference's public calls
    (``add_request`` / ``step``, src/miniserve/engine.py:143-205, paged_engine.py:57-66). ``kind``: "graphs" is its
    ``Engine(cuda_graphs=True)`` on the slot cache (its fastest decode, docs/RESULTS.md:38-40), "paged" its ``PagedEngine``."""
    from miniserve.engine import Engine, Request
    from miniserve.paged_engine import PagedEngine

    total = steps + warmup + 8
    prompt_len = CONTEXT - total
    max_len = CONTEXT + 8
    if kind == "graphs":
        eng = Engine(model, max_slots=batch, max_len=max_len, policy="continuous", max_prefills_per_step=batch, cuda_graphs=True)
    else:
        per_seq = -(-max_len // BLOCK)
        eng = PagedEngine(model, num_blocks=batch * (per_seq + 1) + 1, block_size=BLOCK, max_seqs=batch, max_len=max_len,
                          enable_prefix_cache=False, max_prefills_per_step=batch)
    g = torch.Generator().manual_seed(9)
    reqs = [eng.add_request(Request(torch.randint(0, MODEL["vocab_size"], (prompt_len,), generator=g).tolist(), max_new_tokens=total))
            for _ in range(batch)]
    t0 = time.perf_counter()
    eng.step()  # admits and prefills every request (one forward each), no decode yet
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    assert len(eng.running) == batch, f"the reference admitted {len(eng.running)} of {batch} requests"
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    before = sum(len(r.output_ids) for r in reqs)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    for _ in range(steps):
        eng.step()
    stop.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    made = sum(len(r.output_ids) for r in reqs) - before
    ms = start.elapsed_time(stop) / steps
    del eng
    torch.cuda.empty_cache()
    return {"ms": ms, "tok_s": made / (ms * steps) * 1e3, "e2e_tok_s": made / wall, "e2e_ms": wall / steps * 1e3,
            "prefill_s": round(prefill_s, 2), "made": made}


def _reference_prefill(model, torch, reps: int = 5) -> dict:
    from miniserve.paged_engine import PagedEngine
    from miniserve.engine import Request

    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, MODEL["vocab_size"], (PREFILL_TOKENS,), generator=g).tolist()
    eng = PagedEngine(model, num_blocks=PREFILL_TOKENS // BLOCK + 4, block_size=BLOCK, max_seqs=1, max_len=PREFILL_TOKENS + 1,
                      enable_prefix_cache=False)
    times = []
    for i in range(reps + 3):
        eng.add_request(Request(prompt, max_new_tokens=1))
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        eng.step()  # prefill of the whole prompt and its first token; the request ends with it
        stop.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(start.elapsed_time(stop))
    return {"ms": sorted(times)[len(times) // 2]}


def reference_arm(a) -> int:
    """The reference itself, unmodified, for the same metric: its model class and its engines from ``baseline/_ref`` (a copy
    of its pure-Python package ``src/miniserve``: what installing its wheel puts into a target folder; building that
    wheel needs the backend ``hatchling``, which the offline wheelhouse lacks). Nothing of this repository's engine, model or
    kernels is on this path; only the writer of the random-weights folder is shared, so that both arms load the same file."""
    if not (REF_DIR / "miniserve" / "paged_engine.py").is_file():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/miniserve (the unmodified copy of the reference's package) is not there"}))
        return 0
    if a.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "the reference runs on one GPU only"}))
        return 0
    sys.path.insert(0, str(REF_DIR))
    import torch

    from llm_infrence_engine_b200.weights import write_random_model  # the folder writer only

    steps, warmup = a.steps, max(a.warmup, 3)
    pk = peaks()
    sampler = ClockSampler()
    try:
        with tempfile.TemporaryDirectory() as tmp:
            folder = write_random_model(dict(MODEL), Path(tmp) / "model", seed=0, store_dtype="bfloat16")
            model = _reference_model(folder, torch)
        sampler.start()
        runs = {}
        for kind in ("graphs", "paged"):
            try:
                runs[kind] = _reference_decode(model, torch, kind, a.batch, steps, warmup)
            except Exception as e:  # one of its two engines failing leaves the other
                runs[kind] = {"error": f"{type(e).__name__}: {e}"[:300]}
        clocks = sampler.stop()
        ok = {k: v for k, v in runs.items() if "error" not in v}
        if not ok:
            print(json.dumps({"impl": "reference", "unavailable": "both of the reference's engines failed: " + json.dumps(runs)}))
            return 0
        best = max(ok, key=lambda k: ok[k]["tok_s"])
        main_pt = ok[best]
        points = {}
        for name, b, n in (("decode_b1", 1, min(steps, 64)), ("decode_b64", 64, min(steps, 16))):
            try:
                points[name] = round(_reference_decode(model, torch, "paged" if b > 8 else best, b, n, 3)["tok_s"], 1)
            except Exception as e:
                points[name] = None
                points[name + "_error"] = f"{type(e).__name__}: {e}"[:200]
        try:
            pre = _reference_prefill(model, torch)
        except Exception as e:
            pre = None
            points["prefill_error"] = f"{type(e).__name__}: {e}"[:200]
    finally:
        if sampler.proc is not None and sampler.proc.poll() is None:
            sampler.stop()
    fl = flops_prefill(PREFILL_TOKENS)
    cache_bytes = a.batch * CONTEXT * MODEL["num_hidden_layers"] * 2 * MODEL["num_key_value_heads"] * 64 * 2
    weight_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
    achieved = (weight_bytes + cache_bytes) / (main_pt["ms"] * 1e-3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {a.batch}, context {CONTEXT} (Qwen2.5-0.5B shape, bf16, random weights)",
        "value": round(main_pt["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(main_pt["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights (seed 0), uniform random token ids; contexts filled by the reference's own prefill",
        "impl": "reference",
        "config": {"model": "Qwen2.5-0.5B shape", "layers": MODEL["num_hidden_layers"], "layers_of_model": MODEL["num_hidden_layers"],
                   "hidden": MODEL["hidden_size"], "heads": MODEL["num_attention_heads"], "kv_heads": MODEL["num_key_value_heads"],
                   "head_dim": 64, "intermediate": MODEL["intermediate_size"], "vocab": MODEL["vocab_size"], "tied": True,
                   "global_batch": a.batch, "seq_len": CONTEXT, "block_size": BLOCK, "parallelism": "single GPU",
                   "cuda_graphs": best == "graphs", "engine": "Engine(cuda_graphs=True), slot cache" if best == "graphs" else "PagedEngine",
                   "l2": "inputs larger than L2 (weights + cache per step >> 126 MB), no flush", "peaks": pk["source"]},
        "clocks": clocks,
        "gpu_launches": 0,
        "engines": {k: ({"tok_s": round(v["tok_s"], 1), "ms_per_step": round(v["ms"], 3), "prefill_s": v["prefill_s"]} if "error" not in v else v)
                    for k, v in runs.items()},
        "prefill": None if pre is None else {"value": round(PREFILL_TOKENS / (pre["ms"] * 1e-3), 1), "tokens": PREFILL_TOKENS,
                                             "ms": round(pre["ms"], 3), "frac": round(fl / (pre["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "e2e": {"value": round(main_pt["e2e_tok_s"], 2), "unit": "tokens/s", "h2d_bytes_per_step": 16 * a.batch, "d2h_bytes_per_step": 8 * a.batch,
                "ms_per_step": round(main_pt["e2e_ms"], 3), "prefill_s": main_pt["prefill_s"]},
    }
    print(json.dumps(line))
    return 0


def check_decode_step(runner, entries, graph_logits, graph_tokens, torch) -> dict:
    """Outside the timed region: is what the captured step computes right?

    (a) The attention of this very shape (these block tables, contexts and pools, the planner's own number of key slices
    and way of merging them) against another kernel altogether: the generic one (one thread per key, 32-bit arithmetic,
    slices at fixed places), on random queries. Bound: 1e-2 of the largest output, the bound of the kernels' own tests.
    (b) The whole step again eagerly, kernel by kernel, and with the generic attention. The logits of two runs of the
    same bfloat16 step are not bit-equal: split-K partial sums meet by atomic additions in whatever order they arrive, the
    last bits of a sum decide how some activations round to bfloat16, and a deep model with random weights carries such
    a flip through to the logits (two replays of one graph were measured 1e-2 of the logits' scale apart at 24 layers, 1e-3
    at 2, and exactly equal with split-K off). So (b) is a coarse bound, 4e-2 of the scale, and the graph's tokens must be
    the eager argmax wherever the two best logits are clearly apart."""
    K = runner.K
    ctx, rows = runner.make_context(entries)
    eager = runner.forward(ctx, rows).float()
    slices = int(K.last_attention_plan[0])
    mixer = runner.spec.layers[runner.spec.schedule[0].layer].mixer
    bind = runner.bindings[runner.spec.schedule[0].cache]
    g = torch.Generator(device="cuda").manual_seed(3)
    width = (mixer.num_heads + 2 * mixer.num_kv_heads) * mixer.head_dim
    qkv = torch.randn((ctx.num_tokens, width), generator=g, device="cuda").to(torch.bfloat16)
    args = (qkv, bind.k, bind.v, ctx.block_tables[bind.group], ctx.token_seq, ctx.positions, mixer.num_heads, mixer.num_kv_heads,
            mixer.head_dim, ctx.page_size, mixer.scale, mixer.window or 0, ctx.max_context)
    fast = K.paged_attention(*args, batch=ctx).float()
    plain = K.paged_attention(*args).float()   # without the step's description the generic kernel runs
    d_attn = float((fast - plain).abs().max()) / max(float(plain.abs().max()), 1e-30)
    ctx._tables.clear()
    was = K.use_mma_attention
    K.use_mma_attention = False
    try:
        generic = runner.forward(ctx, rows).float()
    finally:
        K.use_mma_attention = was
    scale = max(1.0, float(eager.abs().max()))
    d_eager = float((graph_logits - eager).abs().max()) / scale
    d_generic = float((graph_logits - generic).abs().max()) / scale
    top2 = eager.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 4 * float((graph_logits - eager).abs().max())
    same = graph_tokens.long() == eager.argmax(-1)
    ok = bool(d_attn <= 1e-2 and d_eager <= 4e-2 and d_generic <= 4e-2 and bool((same | ~clear).all())
              and bool(torch.isfinite(graph_logits).all()))
    return {"checked": ok, "attention_vs_generic_kernel": round(d_attn, 5), "graph_vs_eager": round(d_eager, 5),
            "vs_generic_attention": round(d_generic, 5), "tokens_equal": int(same.sum()), "rows": int(same.numel()),
            "attention_slices": slices}


def decode_point(folder: Path, batch: int, steps: int, warmup: int, torch, graphs: bool = True, sampler=None) -> dict:
    """Device time of ``steps`` decode steps of ``batch`` requests at CONTEXT tokens: the step function
    (replayed from its CUDA graph unless ``graphs`` is off) plus the argmax over its logits."""
    from llm_infrence_engine_b200.config import EngineConfig
    from llm_infrence_engine_b200.engine import StepEntry, build_runner

    per_seq = -(-(CONTEXT + 8) // BLOCK)
    cfg = EngineConfig(dtype="bfloat16", block_size=BLOCK, num_blocks=batch * per_seq + 1, max_seqs=batch, max_len=CONTEXT + 8,
                       max_num_batched_tokens=max(batch, 16), cuda_graphs=graphs)
    spec, cache, runner = build_runner(folder, cfg)
    K = runner.K
    for b in runner.bindings:
        b.k.normal_(0, 0.5)
        b.v.normal_(0, 0.5)
    entries = []
    for i in range(batch):
        cache.admit(i)
        cache.reserve(i, 0, CONTEXT)
        entries.append(StepEntry(i, [(17 * i + 3) % MODEL["vocab_size"]], CONTEXT - 1, (0,)))
    check = None
    if graphs:
        runner.step(entries)  # captures the graph for this batch size and leaves the step's inputs in its static buffer
        cap = runner.graphs.captured[batch]
        per_step = cap.launches  # the captured step ends with the argmax over its logits
        check = check_decode_step(runner, entries, cap.logits[:batch].clone(), cap.tokens[:batch].clone(), torch)

        def one():
            cap.graph.replay()
            return cap.tokens
    else:
        ctx, rows = runner.make_context(entries)
        n0 = K.launches

        def one():
            ctx._tables.clear()
            return K.argmax(runner.forward(ctx, rows))

        one()
        per_step = K.launches - n0

    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.start()
        for _ in range(min(steps, 200)):  # bring the clocks up before the samples count
            one()
        torch.cuda.synchronize()
        sampler.rows.clear()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        one()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    if sampler is not None:
        sampler.clocks = sampler.stop()
    K.check_device_errors()  # a kernel that gave up on a bounded wait would have left invalid logits behind
    out = {"ms": ms, "tok_s": batch / ms * 1e3, "launches": per_step * steps, "check": check,
           "bytes": runner.weight_bytes_per_step() + batch * CONTEXT * runner.kv_bytes_per_token}
    del runner, spec, cache
    torch.cuda.empty_cache()
    return out


def prefill_point(folder: Path, torch, reps: int = 5, graphs: bool = True) -> dict:
    from llm_infrence_engine_b200.config import EngineConfig
    from llm_infrence_engine_b200.engine import StepEntry, build_runner

    cfg = EngineConfig(dtype="bfloat16", block_size=BLOCK, num_blocks=PREFILL_TOKENS // BLOCK + 2, max_seqs=1,
                       max_len=PREFILL_TOKENS, max_num_batched_tokens=PREFILL_TOKENS, cuda_graphs=graphs)
    spec, cache, runner = build_runner(folder, cfg)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, MODEL["vocab_size"], (PREFILL_TOKENS,), generator=g).tolist()
    times = []
    for i in range(reps + 3):  # the first three runs are warm-up: with graphs the step's shape is captured at its third coming
        cache.admit("p")
        cache.reserve("p", 0, PREFILL_TOKENS)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry("p", prompt, 0, (PREFILL_TOKENS - 1,))])
        stop.record()
        torch.cuda.synchronize()
        cache.free("p")
        if i >= 3:
            times.append(start.elapsed_time(stop))
    ms = sorted(times)[len(times) // 2]
    del runner, spec, cache
    torch.cuda.empty_cache()
    return {"ms": ms}


def e2e_point(folder: Path, batch: int, steps: int, warmup: int, torch, graphs: bool = True) -> dict:
    """``Engine.step()`` in a loop: host token lists in, sampled tokens out, after the engine prefilled the prompts itself."""
    from llm_infrence_engine_b200.engine import Engine, Request

    total = steps + warmup + 96  # nobody finishes before the timed steps, even the request that was admitted first
    prompt_len = CONTEXT - total
    per_seq = -(-(CONTEXT + 8) // BLOCK)
    eng = Engine(str(folder), dtype="bfloat16", block_size=BLOCK, num_blocks=batch * per_seq + 1, max_seqs=batch,
                 max_len=CONTEXT + 8, max_num_batched_tokens=2048, cuda_graphs=graphs, pipeline=True)
    g = torch.Generator().manual_seed(9)
    reqs = [eng.add_request(Request(torch.randint(0, MODEL["vocab_size"], (prompt_len,), generator=g).tolist(), max_new_tokens=total))
            for _ in range(batch)]
    t0 = time.perf_counter()
    while any(r.num_computed < prompt_len for r in reqs) or any(len(r.output_ids) < 1 for r in reqs):
        eng.step()
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    before = sum(len(r.output_ids) for r in reqs)
    t0 = time.perf_counter()
    for _ in range(steps):
        eng.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    made = sum(len(r.output_ids) for r in reqs) - before
    h2d = eng.runner.last_h2d_bytes
    return {"value": made / dt, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * batch,
            "ms_per_step": dt / steps * 1e3, "prefill_s": round(prefill_s, 2)}


def serving_point(folder: Path, torch, n_requests: int, seed: int, budget: int, passes: int = 2) -> dict:
    """Continuous batching of ``n_requests`` requests that all arrive at once: prompt lengths uniform in [128, 2048], output
    lengths uniform in [64, 512] (seeded), through ``Engine`` with graphs captured up front (``warmup()``), the pipelined
    engine and a token budget per step. The workload is run ``passes`` times on fresh engines; the last pass counts (the
    first also pays for loading the CUDA library and the first captures). The reference's counterpart is its burst benchmark
    (benchmarks/bench_batching.py: every request at once, throughput = generated tokens / wall time)."""
    import random

    from llm_infrence_engine_b200.engine import Engine, Request

    rng = random.Random(seed)
    spec = [(rng.randint(128, 2048), rng.randint(64, 512)) for _ in range(n_requests)]
    max_len = 2048 + 512 + 16
    out = None
    for _ in range(passes):
        eng = Engine(str(folder), dtype="bfloat16", block_size=BLOCK, max_seqs=n_requests, max_len=max_len,
                     num_blocks=n_requests * (-(-max_len // BLOCK)) + 1, max_num_batched_tokens=budget, cuda_graphs=True, pipeline=True)
        t0 = time.perf_counter()
        eng.warmup()
        torch.cuda.synchronize()
        warm_s = time.perf_counter() - t0
        g = torch.Generator().manual_seed(seed + 1)
        reqs = [eng.add_request(Request(torch.randint(0, MODEL["vocab_size"], (p,), generator=g).tolist(), max_new_tokens=o, ignore_eos=True))
                for p, o in spec]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.run_until_idle()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        made = sum(len(r.output_ids) for r in reqs)
        prompt = sum(p for p, _ in spec)
        dec = [s for s in eng.steps if s.num_prefill_tokens == 0 and s.decode_batch]
        mix = [s for s in eng.steps if s.num_prefill_tokens > 0]
        ttft = sorted((r.first_token_time - r.arrival_time) for r in reqs if r.first_token_time is not None)
        out = {"output_tok_s": round(made / dt, 1), "total_tok_s": round((made + prompt) / dt, 1), "wall_s": round(dt, 3),
               "requests": n_requests, "prompt_tokens": prompt, "output_tokens": made, "steps": len(eng.steps),
               "decode_only_steps": len(dec), "decode_only_ms": round(1e3 * sum(s.duration for s in dec) / max(1, len(dec)), 3),
               "mean_decode_batch": round(sum(s.decode_batch for s in dec) / max(1, len(dec)), 1),
               "steps_with_prompt_tokens": len(mix), "prompt_step_ms": round(1e3 * sum(s.duration for s in mix) / max(1, len(mix)), 3),
               "ttft_mean_s": round(sum(ttft) / max(1, len(ttft)), 3), "ttft_p95_s": round(ttft[int(0.95 * (len(ttft) - 1))], 3) if ttft else None,
               "preemptions": eng.stats()["preemptions"], "graph_warmup_s": round(warm_s, 2), "token_budget": budget}
        assert all(len(r.output_ids) == o for r, (_, o) in zip(reqs, spec))
        del eng
        torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------------------------------------------------
# ``--workload luvutar``: the Luvutar decoder at layer sizes of real models, beside the Qwen2 decoder of equal size.

LUVUTAR_SIZES = {
    # name: (width, heads, kv_heads, head_dim, rot_dim, q_rank, kv_rank, window, ff, streams, layers, vocab)
    "0.5b-like": (896, 14, 2, 64, 32, 384, 256, 1024, 3584, 4, 8, 32768),
    "3b-like": (2048, 16, 4, 128, 64, 768, 512, 2048, 8192, 4, 8, 32768),
}


def luvutar_config(size: str) -> dict:
    """Layers in the order attention, latent attention, attention reading the first one's keys and values, latent attention, ..."""
    W, H, G, d, r, qr, kr, win, ff, streams, layers, vocab = LUVUTAR_SIZES[size]
    out = []
    for i in range(layers):
        if i % 2:
            m = {"heads": H, "dim": d, "rot_dim": r, "vdim": d, "q_rank": qr, "kv_rank": kr, "scale": (d + r) ** -0.5,
                 "mask": {"size": win}, "rot": {"base": 10000.0, "dims": r}}
            out.append({"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff}})
        else:
            m = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5, "bias_max": 4096, "q_temp": {"coef": 0.1, "every": 1024}}
            if i % 4 == 2:
                m["kv_from"] = i - 2
            out.append({"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff}})
    return {"architecture": "Luvutar", "vocab": vocab, "width": W, "norm": {"eps": 1e-6}, "streams": streams, "layers": out}


def qwen2_like(size: str) -> dict:
    """The Qwen2 decoder with the same width, heads, layers and vocabulary, and a gated feed-forward of as many weights."""
    W, H, G, d, r, qr, kr, win, ff, streams, layers, vocab = LUVUTAR_SIZES[size]
    return {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": vocab, "hidden_size": W, "head_dim": d,
            "intermediate_size": (2 * ff // 3 + 127) // 128 * 128, "num_hidden_layers": layers, "num_attention_heads": H,
            "num_key_value_heads": G, "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "tie_word_embeddings": False,
            "max_position_embeddings": 32768, "use_sliding_window": False, "hidden_act": "silu"}


def model_points(folder: Path, vocab: int, batch: int, context: int, prefill_tokens: int, steps: int, warmup: int, torch) -> dict:
    """Decode steps (``batch`` requests at ``context`` tokens, replayed from a CUDA graph, argmax included) and one prompt of
    ``prefill_tokens`` tokens, both as device time between two events; launches of a step and the bytes it must read."""
    from llm_infrence_engine_b200.config import EngineConfig
    from llm_infrence_engine_b200.engine import StepEntry, build_runner

    per_seq = -(-(context + 8) // BLOCK)
    cfg = EngineConfig(dtype="bfloat16", block_size=BLOCK, num_blocks=batch * per_seq + 1, max_seqs=batch, max_len=context + 8,
                       max_num_batched_tokens=max(batch, 16), cuda_graphs=True)
    spec, cache, runner = build_runner(folder, cfg)

    def fill(b):   # synthetic cache contents; states of fixed size keep their zeros
        if isinstance(b, tuple):
            for x in b:
                fill(x)
        elif hasattr(b, "k"):
            b.k.normal_(0, 0.5)
            if b.v is not None:
                b.v.normal_(0, 0.5)

    for b in runner.bindings:
        fill(b)
    entries = []
    for i in range(batch):
        cache.admit(i)
        cache.reserve(i, 0, context)
        entries.append(StepEntry(i, [(17 * i + 3) % vocab], context - 1, (0,)))
    runner.step(entries)
    cap = runner.graphs.captured[batch]
    for _ in range(warmup):
        cap.graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        cap.graph.replay()
    stop.record()
    torch.cuda.synchronize()
    runner.K.check_device_errors()
    dec_ms = start.elapsed_time(stop) / steps
    from llm_infrence_engine_b200.cache.spec import FixedStateSpec, flatten_specs

    def live(g):   # bytes of one request's cache entry that a decode step reads (a state of fixed size is also written back)
        if isinstance(g, FixedStateSpec):
            n = 1
            for d in g.shape:
                n *= d
            return 2 * 4 * n
        seen = min(context, getattr(g, "window", None) or context)
        if getattr(g, "chunk", None):
            seen = min(seen, (context - 1) % g.chunk + 1)
        if getattr(g, "window", None):
            seen = min(context, seen + getattr(g, "keep_first", 0))
        return 2 * seen * g.num_kv_heads * (g.head_dim + (g.head_dim if g.v_head_dim is None else g.v_head_dim))

    held = sum(live(g) for cs in spec.cache_specs() for g in flatten_specs(cs))
    out = {"decode_ms": round(dec_ms, 4), "decode_tok_s": round(batch / dec_ms * 1e3, 1), "launches_per_step": cap.launches,
           "decode_bytes": runner.weight_bytes_per_step() + batch * held}
    del runner, spec, cache, cap
    torch.cuda.empty_cache()
    cfg = EngineConfig(dtype="bfloat16", block_size=BLOCK, num_blocks=prefill_tokens // BLOCK + 2, max_seqs=1, max_len=prefill_tokens,
                       max_num_batched_tokens=prefill_tokens, cuda_graphs=False)
    spec, cache, runner = build_runner(folder, cfg)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, vocab, (prefill_tokens,), generator=g).tolist()
    times = []
    for i in range(8):
        cache.admit("p")
        cache.reserve("p", 0, prefill_tokens)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry("p", prompt, 0, (prefill_tokens - 1,))])
        stop.record()
        torch.cuda.synchronize()
        cache.free("p")
        if i >= 3:
            times.append(start.elapsed_time(stop))
    runner.K.check_device_errors()
    ms = sorted(times)[len(times) // 2]
    out.update(prefill_ms=round(ms, 3), prefill_tok_s=round(prefill_tokens / ms * 1e3, 1))
    del runner, spec, cache
    torch.cuda.empty_cache()
    return out


def _time(fn, torch, reps: int = 20, warm: int = 3) -> float:
    """Median-free mean device time of ``fn`` in microseconds: warm-up, then ``reps`` calls between two events."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / reps * 1e3


def _time_graph(fn, torch, reps: int = 20) -> float:
    """Device time of ``fn`` in microseconds with the host out of the way: ``reps`` calls are captured in a CUDA graph, and the
    graph's replays are timed (a kernel of a few microseconds is otherwise hidden behind the Python that launches it)."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        fn()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(reps):
                fn()
    torch.cuda.synchronize()
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(3):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / (3 * reps) * 1e3


def luvutar_kernel_points(torch, pk) -> dict:
    """Luvutar's kernels one by one at the 3b-like layer sizes, each beside the Qwen2 kernel that does the like job at the same
    size: microseconds, and the fraction of its roofline (bytes that must move / copy peak, or flops / bf16 peak). Inputs are
    larger than L2 where the kernel streams memory (cache pools of several hundred MB; activations of 2,048 rows are not)."""
    from types import SimpleNamespace

    from llm_infrence_engine_b200.csrc import get_kernels
    from llm_infrence_engine_b200.parts.attention_biased import distance_rows

    K = get_kernels()
    W, H, G, d, r, qr, kr, win, ff, S, _, _ = LUVUTAR_SIZES["3b-like"]
    bf, dev = torch.bfloat16, "cuda"
    hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    out = {}

    def entry(us, bytes_=None, flops=None):
        e = {"us": round(us, 2)}
        if bytes_ is not None:
            e["frac_of_copy_peak"] = round(bytes_ / (us * 1e-6) / hbm, 4)
        if flops is not None:
            e["frac_of_bf16_peak"] = round(flops / (us * 1e-6) / tf, 4)
        return e

    def batch_of(lens):
        starts = [0]
        for n in lens:
            starts.append(starts[-1] + n)
        return SimpleNamespace(seq_lens=list(lens), seq_starts_dev=torch.tensor(starts, dtype=torch.int32, device=dev),
                               max_seq_len=max(lens), _tables={})

    def tables(batch, ctx, page=BLOCK):
        per = -(-ctx // page)
        t = torch.zeros((batch + 1, per), dtype=torch.int32, device=dev)
        t[:batch] = (torch.randperm(batch * per, device=dev).to(torch.int32) + 1).view(batch, per)
        return t, batch * per + 1

    rel = torch.randn(32, H, device=dev)
    rows_of = torch.tensor(distance_rows(32, 4096.0), dtype=torch.int32, device=dev)
    sink = torch.randn(H, device=dev)
    for what, batch, ctx, T in (("decode", 8, 4096, 1), ("decode_b64", 64, 4096, 1), ("prefill", 1, 2048, 2048)):
        table, pages = tables(batch, ctx)
        N = batch * T
        seq = torch.arange(batch, dtype=torch.int32, device=dev).repeat_interleave(T)
        pos = (torch.arange(T, dtype=torch.int32, device=dev) + (ctx - T)).repeat(batch)
        b = batch_of([T] * batch)
        # grouped attention: Qwen2's kernels against the kernel with temperature, distance bias and a gate per head
        kp = torch.randn(pages, G, BLOCK, d, device=dev).to(bf)
        vp = torch.randn(pages, G, BLOCK, d, device=dev).to(bf)
        qkv = torch.randn(N, (H + 2 * G) * d + 8 * ((H + 7) // 8), device=dev).to(bf)
        if T == 1:
            moved, fl = batch * ctx * 2 * G * d * 2, None
        else:
            moved, fl = None, 4.0 * H * d * (T * (T + 1) / 2) * batch
        out[f"attention_{what}_qwen2"] = entry(_time(lambda: (b._tables.clear(), K.paged_attention(qkv, kp, vp, table, seq, pos, H, G, d, BLOCK, d ** -0.5, 0, ctx, batch=b)), torch), moved, fl)
        out[f"attention_{what}_luvutar"] = entry(_time(lambda: (b._tables.clear(), K.attention_ext(qkv, 0, H, G, d, d, kp, vp, table, seq, pos, BLOCK, d ** -0.5, 0, ctx, temp=(0.1, 1024), rel=rel, rel_rows=rows_of,
                                                                                     gate=qkv, gate_col=(H + 2 * G) * d, gate_per_head=True, batch=b)), torch), moved, fl)
        del kp, vp
        # latent attention: one key/value head of kv_rank + rot_dim entries, a window, a sink
        lp = torch.randn(pages, 1, BLOCK, kr + r, device=dev).to(bf)
        ql = torch.randn(N, H * (kr + r), device=dev).to(bf)
        seen = min(win, ctx)
        if T == 1:
            moved, fl = batch * seen * (kr + r) * 2, None
        else:
            moved, fl = None, 2.0 * H * (2 * kr + r) * sum(min(p + 1, win) for p in range(ctx - T, ctx)) * batch
        out[f"latent_attention_{what}_luvutar"] = entry(_time(lambda: (b._tables.clear(), K.attention_ext(ql, 0, H, 1, kr + r, kr, lp, None, table, seq, pos, BLOCK, 0.07, win, ctx, sink=sink, batch=b)), torch), moved, fl)
        del lp
    # norms at 2,048 rows: add + norm of one stream against update + weighted sum + norm of four
    N = 2048
    res, delta, w = torch.randn(N, W, device=dev), torch.randn(N, W, device=dev).to(bf), torch.ones(W, device=dev)
    xs, mix, co, ci = torch.randn(N, S, W, device=dev), torch.eye(S, device=dev), torch.ones(S, device=dev), torch.full((S,), 0.25, device=dev)
    out["norm_qwen2"] = entry(_time(lambda: K.add_rmsnorm(res, delta, w, 1e-6, bf), torch), N * W * (4 + 4 + 2 + 2))

    def hyper():
        K.streams_update(xs, delta, mix, co)
        return K.streams_norm(xs, ci, w, 1e-6, bf)

    out["norm_luvutar"] = entry(_time(hyper, torch), N * W * (8 * S + 2 + 2))
    # feed-forward going in: gate/up product with SiLU against up product with GELU (equal weights: ff against 2 * (2 ff / 3))
    h = torch.randn(N, W, device=dev).to(bf)
    inter = (2 * ff // 3 + 127) // 128 * 128
    wgu, wup = torch.randn(2 * inter, W, device=dev).to(bf) * 0.02, torch.randn(ff, W, device=dev).to(bf) * 0.02
    out["ff_in_qwen2"] = entry(_time(lambda: K.gate_up_act(h, wgu, bf), torch), None, 2.0 * N * W * 2 * inter)
    out["ff_in_luvutar"] = entry(_time(lambda: K.linear_act(h, wup, "gelu_tanh", bf), torch), None, 2.0 * N * W * ff)
    # the per-head products around latent attention (no counterpart in Qwen2)
    q = torch.randn(N, H * (d + r), device=dev).to(bf)
    w_uk, w_uv = torch.randn(H * d, kr, device=dev).to(bf) * 0.05, torch.randn(H, kr, d, device=dev).to(bf) * 0.05
    half = r // 2
    cos, sin = torch.ones(N, half, device=dev), torch.zeros(N, half, device=dev)
    o_lat, gate = torch.randn(N, H * kr, device=dev).to(bf), torch.randn(N, H * d, device=dev).to(bf)
    out["latent_absorb_luvutar"] = entry(_time(lambda: K.latent_absorb(q, w_uk, cos, sin, H, d, r, r, kr), torch), None, 2.0 * N * H * d * kr)
    out["latent_expand_luvutar"] = entry(_time(lambda: K.latent_expand(o_lat, w_uv, gate, 0, H, kr, d), torch), None, 2.0 * N * H * d * kr)
    K.check_device_errors()
    return out


# ``--workload zepalorn``: the Zepalorn decoder at layer sizes of real models, beside the Qwen2 decoder of equal size.

ZEPALORN_SIZES = {
    # name: (width, attention heads, kv heads, head_dim, window, chunk, delta heads, delta key size, delta value size, state-space heads,
    #        state-space value size, state size, state groups, ff, layers, vocab)
    "0.5b-like": (896, 14, 2, 64, 1024, 2048, 8, 64, 128, 28, 64, 128, 2, 2432, 8, 32768),
    "3b-like": (2048, 16, 4, 128, 2048, 4096, 16, 128, 128, 64, 64, 128, 8, 5504, 8, 32768),
}


def zepalorn_config(size: str) -> dict:
    """Layers in the order delta rule, windowed attention, attention beside a state-space mixer, delta rule, ..."""
    W, H, G, d, win, chunk, dh, dd, dv, sh, sv, ns, sg, ff, layers, vocab = ZEPALORN_SIZES[size]
    scaling = {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}
    kinds = []
    for i in range(layers):
        mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
        if i % 4 in (0, 3):
            kinds.append({"type": "channel_delta", "mixer": {"heads": dh, "kv_heads": dh, "dim": dd, "vdim": dv, "conv": 4}, "mlp": mlp})
        elif i % 4 == 1:
            m = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5, "mask": {"size": win, "keep_first": 4},
                 "rot": {"base": 1000000.0, "dims": d, "scaling": scaling}}
            kinds.append({"type": "attention", "mixer": m, "mlp": mlp})
        else:
            left = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5, "conv": 4, "softcap": 50.0, "mask": {"size": chunk},
                    "rot": {"base": 10000.0, "dims": d // 2, "scaling": scaling}}
            right = {"heads": sh, "vdim": sv, "state": ns, "groups": sg, "norm_groups": sg, "conv": 4}
            kinds.append({"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp})
    return {"architecture": "Zepalorn", "vocab": vocab, "width": W, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "layers": kinds}


def qwen2_beside_zepalorn(size: str) -> dict:
    W, H, G, d, win, chunk, dh, dd, dv, sh, sv, ns, sg, ff, layers, vocab = ZEPALORN_SIZES[size]
    return {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": vocab, "hidden_size": W, "head_dim": d,
            "intermediate_size": ff, "num_hidden_layers": layers, "num_attention_heads": H, "num_key_value_heads": G, "rms_norm_eps": 1e-6,
            "rope_theta": 10000.0, "tie_word_embeddings": True, "max_position_embeddings": 32768, "use_sliding_window": False, "hidden_act": "silu"}


def zepalorn_kernel_points(torch, pk) -> dict:
    """Zepalorn's kernels one by one at the 3b-like layer sizes, each beside the Qwen2 kernel that does the like job at the same
    size where there is one: microseconds, and the fraction of its roofline (bytes that must move / copy peak, or flops / bf16
    peak). The recurrences have no tensor-core form here: their flops are set against the bf16 peak all the same, and their bytes
    (state in and out for decoded tokens; projections in, results out for a prompt) against the copy peak."""
    from types import SimpleNamespace

    from llm_infrence_engine_b200.csrc import get_kernels

    K = get_kernels()
    W, H, G, d, win, chunk, dh, dd, dv, sh, sv, ns, sg, ff, _, _ = ZEPALORN_SIZES["3b-like"]
    bf, dev = torch.bfloat16, "cuda"
    hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    out = {}

    def entry(us, bytes_=None, flops=None):
        e = {"us": round(us, 2)}
        if bytes_ is not None:
            e["frac_of_copy_peak"] = round(bytes_ / (us * 1e-6) / hbm, 4)
        if flops is not None:
            e["frac_of_bf16_peak"] = round(flops / (us * 1e-6) / tf, 4)
        return e

    def batch_of(lens, slots=None):
        starts = [0]
        for n in lens:
            starts.append(starts[-1] + n)
        return SimpleNamespace(seq_lens=list(lens), seq_starts_dev=torch.tensor(starts, dtype=torch.int32, device=dev), num_seqs=len(lens),
                               seq_slots=torch.tensor(slots or list(range(len(lens))), dtype=torch.int32, device=dev), max_seq_len=max(lens), _tables={})

    def tables(batch, ctx, page=BLOCK):
        per = -(-ctx // page)
        t = torch.zeros((batch + 1, per), dtype=torch.int32, device=dev)
        t[:batch] = (torch.randperm(batch * per, device=dev).to(torch.int32) + 1).view(batch, per)
        return t, batch * per + 1

    for what, batch, ctx, T in (("decode", 8, 4096, 1), ("decode_b64", 64, 4096, 1), ("prefill", 1, 2048, 2048)):
        table, pages = tables(batch, ctx)
        N = batch * T
        seq = torch.arange(batch, dtype=torch.int32, device=dev).repeat_interleave(T)
        pos = (torch.arange(T, dtype=torch.int32, device=dev) + (ctx - T)).repeat(batch)
        b = batch_of([T] * batch)
        kp = torch.randn(pages, G, BLOCK, d, device=dev).to(bf)
        vp = torch.randn(pages, G, BLOCK, d, device=dev).to(bf)
        qkv = torch.randn(N, (H + 2 * G) * d, device=dev).to(bf)
        if T == 1:
            moved, fl = batch * ctx * 2 * G * d * 2, None
            moved_w, fl_w = batch * (win + 4) * 2 * G * d * 2, None
        else:
            moved, fl = None, 4.0 * H * d * (T * (T + 1) / 2) * batch
            moved_w, fl_w = None, 4.0 * H * d * sum(min(p + 1, win + 4) for p in range(ctx - T, ctx)) * batch
        out[f"attention_{what}_qwen2"] = entry(_time_graph(lambda: (b._tables.clear(), K.paged_attention(qkv, kp, vp, table, seq, pos, H, G, d, BLOCK, d ** -0.5, 0, ctx, batch=b)), torch), moved, fl)
        out[f"attention_{what}_qwen2_window"] = entry(_time_graph(lambda: (b._tables.clear(), K.paged_attention(qkv, kp, vp, table, seq, pos, H, G, d, BLOCK, d ** -0.5, win, ctx, batch=b)), torch), moved_w, fl_w)
        out[f"attention_{what}_zepalorn_window_kept"] = entry(_time_graph(lambda: (b._tables.clear(), K.attention_ext(qkv, 0, H, G, d, d, kp, vp, table, seq, pos, BLOCK, d ** -0.5, win, ctx, batch=b, keep_first=4)), torch), moved_w, fl_w)
        out[f"attention_{what}_zepalorn_chunk_cap"] = entry(_time_graph(lambda: (b._tables.clear(), K.attention_ext(qkv, 0, H, G, d, d, kp, vp, table, seq, pos, BLOCK, d ** -0.5, 0, ctx, batch=b, chunk=chunk, softcap=50.0)), torch), moved, fl)
        del kp, vp
        # the recurrences: state in and out for every request; for a prompt, the projections in and the result out
        qk = torch.randn(N, 2 * dh * dd + dh * dv, device=dev).to(bf) * 0.5
        a_, b_ = torch.randn(N, dh * dd, device=dev).to(bf), torch.randn(N, dh, device=dev).to(bf)
        A_log, dt_bias = torch.zeros(dh, device=dev), torch.full((dh * dd,), -3.0, device=dev)
        state = torch.zeros(batch + 1, dh, dv, dd, device=dev)
        moved = batch * 2 * 4 * dh * dd * dv + N * (2 * (3 * dh * dd + dh * dv) + 4 * dh * dv)
        out[f"delta_rule_{what}_zepalorn"] = entry(_time_graph(lambda: K.delta_rule(qk, dh, dh, dd, dv, a_, b_, 0, A_log, dt_bias, state, b), torch), moved, 8.0 * N * dh * dd * dv)
        xbc = torch.randn(N, sh * sv + 2 * sg * ns, device=dev).to(bf) * 0.5
        dt = torch.randn(N, sh, device=dev).to(bf)
        A2, bias2, skip = torch.zeros(sh, device=dev), torch.full((sh,), -3.0, device=dev), torch.ones(sh, device=dev)
        state2 = torch.zeros(batch + 1, sh, sv, ns, device=dev)
        moved = batch * 2 * 4 * sh * ns * sv + N * (2 * (sh * sv + 2 * sg * ns) + 4 * sh * sv)
        out[f"state_space_{what}_zepalorn"] = entry(_time_graph(lambda: K.ssm_scan(xbc, sh, sg, ns, sv, dt, 0, A2, bias2, skip, state2, b), torch), moved, 6.0 * N * sh * ns * sv)
        C = 2 * dh * dd + dh * dv
        cw, cs = torch.randn(C, 4, device=dev), torch.zeros(batch + 1, 3, C, device=dev)
        out[f"convolution_{what}_zepalorn"] = entry(_time_graph(lambda: K.causal_conv(qk, 0, C, cw, None, cs, b, "silu"), torch), N * C * 4 + batch * C * 3 * 8)
    # norms at 2,048 rows: add + norm of the stream against norm of the result + add + norm of the stream
    N = 2048
    res, delta, w = torch.randn(N, W, device=dev), torch.randn(N, W, device=dev).to(bf), torch.ones(W, device=dev)
    out["norm_qwen2"] = entry(_time_graph(lambda: K.add_rmsnorm(res, delta, w, 1e-6, bf), torch), N * W * (4 + 4 + 2 + 2))

    def both():
        K.post_norm_add(res, delta, w, 1e-6)
        return K.layernorm(res, w, 1e-6, bf)

    out["norm_zepalorn"] = entry(_time_graph(both, torch), N * W * (4 + 4 + 2 + 2))
    # feed-forward going in: the tcgen05 product with SiLU in its epilogue against the same product with the clamped gated unit in it
    h = torch.randn(N, W, device=dev).to(bf)
    wgu = torch.randn(2 * ff, W, device=dev).to(bf) * 0.02
    out["ff_in_qwen2"] = entry(_time_graph(lambda: K.gate_up_act(h, wgu, bf), torch), None, 2.0 * N * W * 2 * ff)
    out["ff_in_zepalorn"] = entry(_time_graph(lambda: K.gate_up_act(h, wgu, bf, glu=(7.0, 1.702, 1.0)), torch), None, 2.0 * N * W * 2 * ff)
    # gated norms of the recurrences' results and the mean of the two halves of a side-by-side mixer (no counterpart in Qwen2)
    o, g = torch.randn(N, dh * dv, device=dev), torch.randn(N, dh * dv, device=dev).to(bf)
    nw = torch.ones(dv, device=dev)
    out["gated_norm_zepalorn"] = entry(_time_graph(lambda: K.group_rmsnorm_gate(o, g, 0, nw, dv, 1e-6, False, bf), torch), N * dh * dv * (4 + 2 + 2))
    a2, b2, y = torch.randn(N, W, device=dev).to(bf), torch.randn(N, W, device=dev).to(bf), torch.zeros(N, W, device=dev)
    out["mean_of_two_zepalorn"] = entry(_time_graph(lambda: K.dual_rmsnorm_mix(a2, b2, w, w, 1e-6, 0.5, y), torch), N * W * (2 + 2 + 4 + 4))
    K.check_device_errors()
    return out


def zepalorn_workload(a) -> int:
    import torch

    from llm_infrence_engine_b200.weights import write_random_model

    pk = peaks()
    sampler = ClockSampler()
    sampler.start()
    sizes = {}
    steps = min(a.steps, 256)
    for size in ZEPALORN_SIZES:
        vocab = ZEPALORN_SIZES[size][-1]
        row = {}
        for name, config in (("zepalorn", zepalorn_config(size)), ("qwen2", qwen2_beside_zepalorn(size))):
            with tempfile.TemporaryDirectory() as tmp:
                folder = write_random_model(config, Path(tmp) / "model", seed=0, store_dtype="bfloat16")
                pt = model_points(folder, vocab, a.batch, a.context or 4096, a.prefill_tokens, steps, max(a.warmup, 3), torch)
            pt["decode_frac_of_copy_peak"] = round(pt["decode_bytes"] / (pt["decode_ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
            row[name] = pt
        sizes[size] = row
    names = ("width", "heads", "kv_heads", "head_dim", "window", "chunk", "delta_heads", "delta_dim", "delta_vdim", "ssm_heads", "ssm_vdim", "ssm_state",
             "ssm_groups", "ff", "layers", "vocab")
    line = {"metric": f"Zepalorn beside Qwen2 of equal size: decode (batch {a.batch}, context {a.context or 4096}) and prefill ({a.prefill_tokens} tokens), bf16, random weights",
            "unit": "ms and tokens/s per size", "n_gpus": 1, "impl": "ours", "dtype": "bf16", "steps": steps, "warmup": max(a.warmup, 3),
            "data": "synthetic: random weights (seed 0), uniform random token ids, synthetic cache contents",
            "config": {"sizes": {k: dict(zip(names, v)) for k, v in ZEPALORN_SIZES.items()}, "block_size": BLOCK, "peaks": pk["source"],
                       "l2": "weights + cache per step larger than L2, no flush"},
            "clocks": sampler.stop(), "sizes": sizes}
    if a.kernels:
        line["kernels"] = zepalorn_kernel_points(torch, pk)
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------------------------------------
# ``--workload mufotar``: the Mufotar decoder at layer sizes of real models, beside the Zepalorn decoder (the closest of the
# engine's other models: delta rule, attention beside a recurrence) of equal width, layers and activated feed-forward size.

MUFOTAR_SIZES = {
    # name: (width, delta heads, delta q/k heads, delta key size, delta value size, attention heads, kv heads, head_dim, scan channels,
    #        scan state, step-size rank, experts, identity experts, chosen, expert ff, shared ff, dense ff, layers, vocab)
    "1b-like": (1024, 8, 4, 128, 128, 8, 2, 128, 2048, 16, 64, 16, 2, 4, 512, 768, 2816, 8, 32768),
    "3b-like": (2048, 16, 8, 128, 128, 16, 4, 128, 4096, 16, 128, 32, 2, 4, 768, 2432, 5504, 8, 32768),
}
MUFOTAR_NAMES = ("width", "delta_heads", "delta_qk_heads", "delta_dim", "delta_vdim", "heads", "kv_heads", "head_dim", "scan_channels", "scan_state",
                 "dt_rank", "experts", "identity_experts", "top", "expert_ff", "shared_ff", "dense_ff", "layers", "vocab")


def mufotar_config(size: str) -> dict:
    """Layers in the order delta rule (dense feed-forward), delta rule, attention beside a selective scan, delta rule (routed
    experts), twice; the second attention layer runs on the first one's weights."""
    W, dh, dg, dd, dv, H, G, d, ci, ns, rk, E, ident, top, eff, sff, ff, layers, vocab = MUFOTAR_SIZES[size]
    moe = {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": E, "identity": ident, "top": top}, "shared": {"ff": sff}}
    delta = {"heads": dh, "kv_heads": dg, "dim": dd, "vdim": dv, "conv": 4}
    pair = {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5, "rot": {"base": 100000.0, "dims": d}},
            "right": {"inner": ci, "state": ns, "dt_rank": rk, "conv": 4}, "left_scale": 1.0, "right_scale": 1.0}
    kinds = []
    for i in range(layers):
        if i % 4 == 2:
            layer = {"type": "parallel", "mixer": pair, "mlp": moe}
            if i > 2:
                layer["weights_of"] = 2
        else:
            layer = {"type": "delta", "mixer": delta, "mlp": {"kind": "dense", "ff": ff} if i % 4 == 0 else moe}
        kinds.append(layer)
    return {"architecture": "Mufotar", "vocab": vocab, "width": W, "norm": {"eps": 1e-6}, "logit_softcap": 30.0, "layers": kinds}


def zepalorn_beside_mufotar(size: str) -> dict:
    """Zepalorn with the same width, layer kinds in the same places (its delta rule has a decay per channel, its recurrence beside
    the attention a state per head), and dense feed-forwards of the size that a Mufotar token activates (chosen experts + shared)."""
    W, dh, dg, dd, dv, H, G, d, ci, ns, rk, E, ident, top, eff, sff, ff, layers, vocab = MUFOTAR_SIZES[size]
    kinds = []
    for i in range(layers):
        mlp = {"kind": "dense", "ff": ff if i % 4 == 0 else top * eff + sff, "limit": 7.0}
        if i % 4 == 2:
            left = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5, "conv": 4, "rot": {"base": 100000.0, "dims": d}}
            right = {"heads": ci // 64, "vdim": 64, "state": 128, "groups": 1, "norm_groups": 1, "conv": 4}
            kinds.append({"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp})
        else:
            kinds.append({"type": "channel_delta", "mixer": {"heads": dh, "kv_heads": dh, "dim": dd, "vdim": dv, "conv": 4}, "mlp": mlp})
    return {"architecture": "Zepalorn", "vocab": vocab, "width": W, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "layers": kinds}


def mufotar_kernel_points(torch, pk) -> dict:
    """Mufotar's kernels one by one at the 3b-like layer sizes, each beside the kernel of the engine's other models that does the
    like job at the same size: microseconds, and the fraction of its roofline (bytes that must move / copy peak, or flops / bf16
    peak). decode: 8 and 64 requests bring one token each; prefill: one request brings 2,048."""
    from types import SimpleNamespace

    from llm_infrence_engine_b200.csrc import get_kernels

    K = get_kernels()
    W, dh, dg, dd, dv, H, G, d, ci, ns, rk, E, ident, top, eff, sff, ff, _, _ = MUFOTAR_SIZES["3b-like"]
    bf, dev = torch.bfloat16, "cuda"
    hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    out = {}

    def entry(us, bytes_=None, flops=None):
        e = {"us": round(us, 2)}
        if bytes_ is not None:
            e["frac_of_copy_peak"] = round(bytes_ / (us * 1e-6) / hbm, 4)
        if flops is not None:
            e["frac_of_bf16_peak"] = round(flops / (us * 1e-6) / tf, 4)
        return e

    def batch_of(lens):
        starts = [0]
        for n in lens:
            starts.append(starts[-1] + n)
        return SimpleNamespace(seq_lens=list(lens), seq_starts_dev=torch.tensor(starts, dtype=torch.int32, device=dev), num_seqs=len(lens),
                               seq_slots=torch.tensor(list(range(len(lens))), dtype=torch.int32, device=dev), max_seq_len=max(lens), _tables={})

    for what, batch, T in (("decode", 8, 1), ("decode_b64", 64, 1), ("prefill", 1, 2048)):
        N = batch * T
        b = batch_of([T] * batch)
        # the delta rule: a decay per head (Mufotar, q/k heads shared by two value heads) beside a decay per channel (Zepalorn)
        qkv = torch.randn(N, 2 * dg * dd + dh * dv, device=dev).to(bf) * 0.5
        z = torch.randn(N, 2 * dh, device=dev).to(bf)
        A_log, bias = torch.zeros(dh, device=dev), torch.full((dh,), -3.0, device=dev)
        state = torch.zeros(batch + 1, dh, dv, dd, device=dev)
        moved = batch * 2 * 4 * dh * dd * dv + N * (2 * (2 * dg * dd + dh * dv) + 4 * dh * dv)
        out[f"delta_rule_{what}_mufotar"] = entry(_time_graph(lambda: K.delta_rule(qkv, dh, dg, dd, dv, z[:, :dh], z, dh, A_log, bias, state, b, decay_per_head=True), torch),
                                                  moved, 8.0 * N * dh * dd * dv)
        qkv2 = torch.randn(N, 2 * dh * dd + dh * dv, device=dev).to(bf) * 0.5
        a2, b2 = torch.randn(N, dh * dd, device=dev).to(bf), torch.randn(N, dh, device=dev).to(bf)
        bias2 = torch.full((dh * dd,), -3.0, device=dev)
        moved = batch * 2 * 4 * dh * dd * dv + N * (2 * (3 * dh * dd + dh * dv) + 4 * dh * dv)
        out[f"delta_rule_{what}_zepalorn"] = entry(_time_graph(lambda: K.delta_rule(qkv2, dh, dh, dd, dv, a2, b2, 0, A_log, bias2, state, b), torch), moved, 8.0 * N * dh * dd * dv)
        # the recurrence beside the attention: a state per channel and index (Mufotar) beside a state per head (Zepalorn)
        x, dt = torch.randn(N, ci, device=dev).to(bf) * 0.5, torch.randn(N, ci, device=dev).to(bf)
        bc, xz = torch.randn(N, rk + 2 * ns, device=dev).to(bf), torch.randn(N, 2 * ci, device=dev).to(bf)
        A2, dtb, skip = torch.zeros(ci, ns, device=dev), torch.full((ci,), -3.0, device=dev), torch.ones(ci, device=dev)
        st = torch.zeros(batch + 1, ci, ns, device=dev)
        moved = batch * 2 * 4 * ci * ns + N * 2 * (4 * ci + 2 * ns)
        out[f"selective_scan_{what}_mufotar"] = entry(_time_graph(lambda: K.selective_scan(x, dt, bc, rk, rk + ns, xz, ci, A2, dtb, skip, st, b), torch), moved, 6.0 * N * ci * ns)
        sh, sv, sn = ci // 64, 64, 128
        xbc, dth = torch.randn(N, sh * sv + 2 * sn, device=dev).to(bf) * 0.5, torch.randn(N, sh, device=dev).to(bf)
        A3, b3, k3 = torch.zeros(sh, device=dev), torch.full((sh,), -3.0, device=dev), torch.ones(sh, device=dev)
        st3 = torch.zeros(batch + 1, sh, sv, sn, device=dev)
        moved = batch * 2 * 4 * sh * sn * sv + N * (2 * (sh * sv + 2 * sn) + 4 * sh * sv)
        out[f"state_space_{what}_zepalorn"] = entry(_time_graph(lambda: K.ssm_scan(xbc, sh, 1, sn, sv, dth, 0, A3, b3, k3, st3, b), torch), moved, 6.0 * N * sh * sn * sv)
        # the feed-forward: router, sort by expert, the experts' two grouped products and the weighted sum (Mufotar) beside a dense
        # gated unit with as many rows of weights as a token's chosen experts have (Zepalorn)
        h = torch.randn(N, W, device=dev).to(bf)
        w_router, corr = torch.randn(E + ident, W, device=dev).to(bf) * 0.05, torch.zeros(E + ident, device=dev)
        wgu, wdn = torch.randn(E, 2 * eff, W, device=dev).to(bf) * 0.02, torch.randn(E, W, eff, device=dev).to(bf) * 0.02
        y = torch.zeros(N, W, device=dev)
        ids, wts = K.moe_router(h, w_router, corr, top)
        real = int((ids < E).sum())
        used = int(torch.unique(ids[ids < E]).numel())
        fl = 6.0 * real * W * eff
        moved = used * 3 * eff * W * 2 + N * W * (2 + 4)
        out[f"router_{what}_mufotar"] = entry(_time_graph(lambda: K.moe_router(h, w_router, corr, top), torch), N * W * 2 + (E + ident) * W * 2)
        out[f"experts_{what}_mufotar"] = entry(_time_graph(lambda: K.moe_experts(h, ids, wts, wgu, wdn, add_to=y), torch), moved, fl)
        wd_gu, wd_dn = torch.randn(2 * top * eff, W, device=dev).to(bf) * 0.02, torch.randn(W, top * eff, device=dev).to(bf) * 0.02
        out[f"dense_unit_{what}_zepalorn"] = entry(_time_graph(lambda: K.linear(K.gate_up_act(h, wd_gu, bf, glu=(7.0, 1.702, 1.0)), wd_dn, add_to=y), torch),
                                                   3 * top * eff * W * 2 + N * W * (2 + 4), 6.0 * N * top * W * eff)
        del wgu, wdn, wd_gu, wd_dn
    # norms, the join of the two mixers, the cap on the logits, at 2,048 rows
    N = 2048
    res, w, bb = torch.randn(N, W, device=dev), torch.ones(W, device=dev), torch.zeros(W, device=dev)
    out["layernorm_bias_mufotar"] = entry(_time_graph(lambda: K.layernorm(res, w, 1e-6, bf, bias=bb), torch), N * W * (4 + 2))
    out["layernorm_zepalorn"] = entry(_time_graph(lambda: K.layernorm(res, w, 1e-6, bf), torch), N * W * (4 + 2))
    a2, b2, y = torch.randn(N, W, device=dev), torch.randn(N, W, device=dev), torch.zeros(N, W, device=dev)
    out["weighted_pair_mufotar"] = entry(_time_graph(lambda: K.weighted_pair(a2, b2, 1.3, 0.7, y), torch), N * W * (4 + 4 + 4 + 4))
    out["mean_of_two_zepalorn"] = entry(_time_graph(lambda: K.dual_rmsnorm_mix(a2, b2, w, w, 1e-6, 0.5, y), torch), N * W * (4 + 4 + 4 + 4))
    o, g, nw = torch.randn(N, dh * dv, device=dev), torch.randn(N, dh * dv, device=dev).to(bf), torch.ones(dv, device=dev)
    out["gated_norm_silu_mufotar"] = entry(_time_graph(lambda: K.group_rmsnorm_gate(o, g, 0, nw, dv, 1e-6, False, bf, gate_act="silu"), torch), N * dh * dv * (4 + 2 + 2))
    out["gated_norm_zepalorn"] = entry(_time_graph(lambda: K.group_rmsnorm_gate(o, g, 0, nw, dv, 1e-6, False, bf), torch), N * dh * dv * (4 + 2 + 2))
    lg = torch.randn(64, 32768, device=dev)
    out["softcap_mufotar"] = entry(_time_graph(lambda: K.softcap(lg, 30.0), torch), 64 * 32768 * 8)
    K.check_device_errors()
    return out


def mufotar_workload(a) -> int:
    import torch

    from llm_infrence_engine_b200.weights import write_random_model

    pk = peaks()
    sampler = ClockSampler()
    sampler.start()
    sizes = {}
    steps = min(a.steps, 256)
    for size in MUFOTAR_SIZES:
        W, E, ident, top, eff = (MUFOTAR_SIZES[size][i] for i in (0, 11, 12, 13, 14))
        layers, vocab = MUFOTAR_SIZES[size][-2:]
        row = {}
        for name, config in (("mufotar", mufotar_config(size)), ("zepalorn", zepalorn_beside_mufotar(size))):
            with tempfile.TemporaryDirectory() as tmp:
                folder = write_random_model(config, Path(tmp) / "model", seed=0, store_dtype="bfloat16")
                pt = model_points(folder, vocab, a.batch, a.context or 4096, a.prefill_tokens, steps, max(a.warmup, 3), torch)
            if name == "mufotar":   # a step reads at most batch * top of a layer's experts: the others' matrices are taken off the bytes
                own = sum(1 for lc in config["layers"] if lc["mlp"]["kind"] == "moe" and "weights_of" not in lc)
                pt["decode_bytes"] -= own * max(0, E - a.batch * top) * 3 * eff * W * 2
            pt["decode_frac_of_copy_peak"] = round(pt["decode_bytes"] / (pt["decode_ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
            row[name] = pt
        sizes[size] = row
    line = {"metric": f"Mufotar beside Zepalorn of equal size: decode (batch {a.batch}, context {a.context or 4096}) and prefill ({a.prefill_tokens} tokens), bf16, random weights",
            "unit": "ms and tokens/s per size", "n_gpus": 1, "impl": "ours", "dtype": "bf16", "steps": steps, "warmup": max(a.warmup, 3),
            "data": "synthetic: random weights (seed 0), uniform random token ids, synthetic cache contents",
            "config": {"sizes": {k: dict(zip(MUFOTAR_NAMES, v)) for k, v in MUFOTAR_SIZES.items()}, "block_size": BLOCK, "peaks": pk["source"],
                       "l2": "weights + cache per step larger than L2, no flush"},
            "clocks": sampler.stop(), "sizes": sizes}
    if a.kernels:
        line["kernels"] = mufotar_kernel_points(torch, pk)
    print(json.dumps(line))
    return 0


# ``--workload memilorn``: the Memilorn decoder at layer sizes of real models, beside the Mufotar decoder (the closest of the
# engine's other models: routed experts, a recurrence with a matrix state, softmax attention) of equal width, layer runs and experts.

MEMILORN_SIZES = {
    # name: (width, memory heads, memory key size, memory value size, attention heads, kv heads, head_dim, latent heads, latent head size,
    #        latent rank, experts, chosen, expert ff, shared ff, vocab)
    "1b-like": (1024, 8, 128, 128, 8, 2, 128, 8, 128, 256, 16, 4, 512, 768, 32768),
    "3b-like": (2048, 16, 128, 128, 16, 4, 128, 16, 128, 512, 32, 4, 768, 2432, 32768),
}
MEMILORN_NAMES = ("width", "memory_heads", "memory_dim", "memory_vdim", "heads", "kv_heads", "head_dim", "latent_heads", "latent_head_dim", "kv_rank",
                  "experts", "top", "expert_ff", "shared_ff", "vocab")


def memilorn_config(size: str) -> dict:
    """Five layers (attention whose heads talk, two matrix memories, latent attention, a matrix memory), of which the middle three run
    twice: eight layer runs, every one with routed experts."""
    W, mh, md, mv, H, G, d, lh, ld, rank, E, top, eff, sff, vocab = MEMILORN_SIZES[size]
    moe = {"kind": "moe", "expert": {"ff": eff, "limit": 7.0}, "router": {"experts": E, "top": top}, "shared": {"ff": sff, "limit": 7.0}}
    memory = {"type": "mlstm", "mixer": {"heads": mh, "dim": md, "vdim": mv, "gate_cap": 15.0}, "mlp": moe}
    attention = {"type": "attention", "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5, "softcap": 30.0,
                                                "rot": {"base": 100000.0, "dims": d}}, "mlp": moe}
    latent = {"type": "latent_attention", "mixer": {"heads": lh, "dim": ld, "vdim": ld, "kv_rank": rank, "scale": ld ** -0.5}, "mlp": moe}
    return {"architecture": "Memilorn", "vocab": vocab, "width": W, "norm": {"eps": 1e-6}, "layers": [attention, memory, memory, latent, memory],
            "loop": {"start": 1, "stop": 4, "times": 2}}


def mufotar_beside_memilorn(size: str) -> dict:
    """Mufotar with the same width and eight layers in the like places: the delta rule (a decay per head) where Memilorn has a matrix
    memory, attention beside a selective scan where it has an attention, the same routed experts in every layer."""
    W, mh, md, mv, H, G, d, lh, ld, rank, E, top, eff, sff, vocab = MEMILORN_SIZES[size]
    moe = {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": E, "identity": 0, "top": top}, "shared": {"ff": sff}}
    delta = {"type": "delta", "mixer": {"heads": mh, "kv_heads": mh, "dim": md, "vdim": mv, "conv": 4}, "mlp": moe}
    pair = {"type": "parallel", "mixer": {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": d ** -0.5, "rot": {"base": 100000.0, "dims": d}},
                                          "right": {"inner": 2 * W, "state": 16, "dt_rank": W // 16, "conv": 4}, "left_scale": 1.0, "right_scale": 1.0}, "mlp": moe}
    return {"architecture": "Mufotar", "vocab": vocab, "width": W, "norm": {"eps": 1e-6}, "layers": [pair, delta, delta, pair, delta, delta, pair, delta]}


def memilorn_kernel_points(torch, pk) -> dict:
    """Memilorn's kernels one by one at the 3b-like layer sizes, each beside the kernel of the engine's other models that does the like
    job at the same size: microseconds, and the fraction of its roofline (bytes that must move / copy peak, or flops / bf16 peak).
    decode: 8 and 64 requests at 4,096 tokens bring one token each; prefill: one request brings 2,048."""
    from types import SimpleNamespace

    from llm_infrence_engine_b200.csrc import get_kernels

    K = get_kernels()
    W, mh, md, mv, H, G, d, lh, ld, rank, E, top, eff, sff, _ = MEMILORN_SIZES["3b-like"]
    bf, dev = torch.bfloat16, "cuda"
    hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    out = {}

    def entry(us, bytes_=None, flops=None):
        e = {"us": round(us, 2)}
        if bytes_ is not None:
            e["frac_of_copy_peak"] = round(bytes_ / (us * 1e-6) / hbm, 4)
        if flops is not None:
            e["frac_of_bf16_peak"] = round(flops / (us * 1e-6) / tf, 4)
        return e

    def batch_of(lens):
        starts = [0]
        for n in lens:
            starts.append(starts[-1] + n)
        return SimpleNamespace(seq_lens=list(lens), seq_starts_dev=torch.tensor(starts, dtype=torch.int32, device=dev), num_seqs=len(lens),
                               seq_slots=torch.tensor(list(range(len(lens))), dtype=torch.int32, device=dev), max_seq_len=max(lens), _tables={})

    def tables(batch, ctx, page=BLOCK):
        per = -(-ctx // page)
        t = torch.zeros((batch + 1, per), dtype=torch.int32, device=dev)
        t[:batch] = (torch.randperm(batch * per, device=dev).to(torch.int32) + 1).view(batch, per)
        return t, batch * per + 1

    for what, batch, ctx, T in (("decode", 8, 4096, 1), ("decode_b64", 64, 4096, 1), ("prefill", 1, 2048, 2048)):
        N = batch * T
        b = batch_of([T] * batch)
        # the recurrence: the matrix memory (scan, then division, norm and gate) beside the delta rule with a decay per head (scan, then
        # norm and gate); both keep heads x key size x value size numbers per request
        z = torch.randn(N, 2 * mh * md + 2 * mh * mv, device=dev).to(bf) * 0.5
        gates = torch.randn(N, 2 * mh, device=dev)
        zero, nw = torch.zeros(mh, device=dev), torch.ones(mh * mv, device=dev)
        S, M = torch.zeros(batch + 1, mh, mv + 1, md, device=dev), torch.zeros(batch + 1, mh, device=dev)
        moved = batch * 2 * 4 * mh * md * (mv + 1) + N * (2 * (2 * mh * md + mh * mv) + 2 * 4 * mh * (mv + 1))
        out[f"matrix_memory_{what}_memilorn"] = entry(_time_graph(lambda: K.mlstm(z, 0, mh * md, 2 * mh * md, gates, zero, zero, 15.0, mh, md, mv, S, M, b), torch),
                                                      moved, 6.0 * N * mh * md * (mv + 1))
        num, mm = K.mlstm(z, 0, mh * md, 2 * mh * md, gates, zero, zero, 15.0, mh, md, mv, S, M, b)
        out[f"memory_finish_{what}_memilorn"] = entry(_time_graph(lambda: K.mlstm_finish(num, mm, z, 2 * mh * md + mh * mv, nw, 1e-6, bf), torch), N * mh * mv * (4 + 2 + 2))
        qkv = torch.randn(N, 2 * mh * md + mh * mv, device=dev).to(bf) * 0.5
        zz = torch.randn(N, 2 * mh, device=dev).to(bf)
        A_log, bias = torch.zeros(mh, device=dev), torch.full((mh,), -3.0, device=dev)
        state = torch.zeros(batch + 1, mh, mv, md, device=dev)
        moved = batch * 2 * 4 * mh * md * mv + N * (2 * (2 * mh * md + mh * mv) + 4 * mh * mv)
        out[f"delta_rule_{what}_mufotar"] = entry(_time_graph(lambda: K.delta_rule(qkv, mh, mh, md, mv, zz[:, :mh], zz, mh, A_log, bias, state, b, decay_per_head=True), torch),
                                                  moved, 8.0 * N * mh * md * mv)
        o, g, nw1 = torch.randn(N, mh * mv, device=dev), torch.randn(N, mh * mv, device=dev).to(bf), torch.ones(mv, device=dev)
        out[f"gated_norm_{what}_mufotar"] = entry(_time_graph(lambda: K.group_rmsnorm_gate(o, g, 0, nw1, mv, 1e-6, False, bf, gate_act="silu"), torch), N * mh * mv * (4 + 2 + 2))
        # attention: heads that talk, with cap, sink and gate (Memilorn) beside plain grouped attention of the same sizes (Mufotar's left half)
        table, pages = tables(batch, ctx)
        seq = torch.arange(batch, dtype=torch.int32, device=dev).repeat_interleave(T)
        pos = (torch.arange(T, dtype=torch.int32, device=dev) + (ctx - T)).repeat(batch)
        kp, vp = torch.randn(pages, G, BLOCK, d, device=dev).to(bf), torch.randn(pages, G, BLOCK, d, device=dev).to(bf)
        q, gt = torch.randn(N, H * d, device=dev).to(bf), torch.randn(N, H, device=dev).to(bf)
        talk, sink = torch.eye(H, device=dev) + 0.05 * torch.randn(H, H, device=dev), torch.zeros(H, device=dev)
        if T == 1:
            moved, fl = batch * ctx * 2 * G * d * 2, None
        else:
            moved, fl = None, 4.0 * H * d * (T * (T + 1) / 2) * batch
        out[f"attention_talk_{what}_memilorn"] = entry(_time_graph(lambda: (b._tables.clear(), K.attention_ext(q, 0, H, G, d, d, kp, vp, table, seq, pos, BLOCK, d ** -0.5, 0, ctx, batch=b,
                                                                                                              softcap=30.0, talk=talk, sink=sink, gate=gt, gate_col=0, gate_per_head=True)), torch), moved, fl)
        out[f"attention_{what}_mufotar"] = entry(_time_graph(lambda: (b._tables.clear(), K.attention_ext(q, 0, H, G, d, d, kp, vp, table, seq, pos, BLOCK, d ** -0.5, 0, ctx, batch=b)), torch), moved, fl)
        del kp, vp
        # latent attention: the attention over the cached latents, one key/value head whose values lie inside its keys (with a gate per head)
        kc = torch.randn(pages, 1, BLOCK, rank, device=dev).to(bf)
        ql = torch.randn(N, lh * rank, device=dev).to(bf)
        if T == 1:
            moved, fl = batch * ctx * rank * 2, None
        else:
            moved, fl = None, 4.0 * lh * rank * (T * (T + 1) / 2) * batch
        out[f"attention_latent_{what}_memilorn"] = entry(_time_graph(lambda: (b._tables.clear(), K.attention_ext(ql, 0, lh, 1, rank, rank, kc, None, table, seq, pos, BLOCK, ld ** -0.5, 0, ctx, batch=b,
                                                                                                                gate=gt, gate_col=0, gate_per_head=True)), torch), moved, fl)
        del kc
        # the feed-forward: sigmoid router, clamped experts with the weight on their input (Memilorn) beside softmax router, SiLU experts (Mufotar)
        h = torch.randn(N, W, device=dev).to(bf)
        w_router, corr = torch.randn(E, W, device=dev).to(bf) * 0.05, torch.zeros(E, device=dev)
        wgu, wdn = torch.randn(E, 2 * eff, W, device=dev).to(bf) * 0.02, torch.randn(E, W, eff, device=dev).to(bf) * 0.02
        y = torch.zeros(N, W, device=dev)
        ids, wts = K.moe_router(h, w_router, None, top, scoring="sigmoid")
        used = int(torch.unique(ids).numel())
        fl = 6.0 * N * top * W * eff
        moved = used * 3 * eff * W * 2 + N * W * (2 + 4)
        out[f"router_{what}_memilorn"] = entry(_time_graph(lambda: K.moe_router(h, w_router, None, top, scoring="sigmoid"), torch), N * W * 2 + E * W * 2)
        out[f"experts_{what}_memilorn"] = entry(_time_graph(lambda: K.moe_experts(h, ids, wts, wgu, wdn, add_to=y, glu=(7.0, 1.702, 1.0), weight_inputs=True), torch), moved, fl)
        ids2, wts2 = K.moe_router(h, w_router, corr, top)
        used2 = int(torch.unique(ids2).numel())
        out[f"router_{what}_mufotar"] = entry(_time_graph(lambda: K.moe_router(h, w_router, corr, top), torch), N * W * 2 + E * W * 2)
        out[f"experts_{what}_mufotar"] = entry(_time_graph(lambda: K.moe_experts(h, ids2, wts2, wgu, wdn, add_to=y), torch), used2 * 3 * eff * W * 2 + N * W * (2 + 4), fl)
        del wgu, wdn
    # the norm of a sublayer's input that also adds the scaled result of the sublayer before (Memilorn) beside the plain norm (Mufotar's has a bias)
    N = 2048
    res, w, bb, ls = torch.randn(N, W, device=dev), torch.ones(W, device=dev), torch.zeros(W, device=dev), torch.ones(W, device=dev)
    delta = torch.randn(N, W, device=dev).to(bf)

    def scaled_then_norm():
        K._pending_post = (res, delta, ls, 0.0, True)
        return K.layernorm(res, w, 1e-6, bf)

    out["norm_with_layer_scale_memilorn"] = entry(_time_graph(scaled_then_norm, torch), N * W * (4 + 4 + 2 + 2))
    out["layernorm_bias_mufotar"] = entry(_time_graph(lambda: K.layernorm(res, w, 1e-6, bf, bias=bb), torch), N * W * (4 + 2))
    ids = torch.randint(0, 32768, (N,), device=dev, dtype=torch.int32)
    table_e = torch.randn(32768, W, device=dev).to(bf)
    out["embedding_added_again_memilorn"] = entry(_time_graph(lambda: K.embed_add(ids, table_e, res), torch), N * W * (2 + 4 + 4))
    K.check_device_errors()
    return out


def memilorn_workload(a) -> int:
    import torch

    from llm_infrence_engine_b200.weights import write_random_model

    pk = peaks()
    sampler = ClockSampler()
    sampler.start()
    sizes = {}
    steps = min(a.steps, 256)
    for size in MEMILORN_SIZES:
        W, E, top, eff, vocab = (MEMILORN_SIZES[size][i] for i in (0, 10, 11, 12, 14))
        row = {}
        for name, config in (("memilorn", memilorn_config(size)), ("mufotar", mufotar_beside_memilorn(size))):
            with tempfile.TemporaryDirectory() as tmp:
                folder = write_random_model(config, Path(tmp) / "model", seed=0, store_dtype="bfloat16")
                pt = model_points(folder, vocab, a.batch, a.context or 4096, a.prefill_tokens, steps, max(a.warmup, 3), torch)
            # a step reads at most batch * top of a layer's experts: the others' matrices are taken off the bytes; a looped layer's weights
            # are counted once per run (they are read again, from L2 or from memory)
            runs = 8
            own = len(config["layers"])
            pt["decode_bytes"] -= own * max(0, E - a.batch * top) * 3 * eff * W * 2
            pt["layer_runs"] = runs
            pt["decode_frac_of_copy_peak"] = round(pt["decode_bytes"] / (pt["decode_ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
            row[name] = pt
        sizes[size] = row
    line = {"metric": f"Memilorn beside Mufotar of equal size: decode (batch {a.batch}, context {a.context or 4096}) and prefill ({a.prefill_tokens} tokens), bf16, random weights",
            "unit": "ms and tokens/s per size", "n_gpus": 1, "impl": "ours", "dtype": "bf16", "steps": steps, "warmup": max(a.warmup, 3),
            "data": "synthetic: random weights (seed 0), uniform random token ids, synthetic cache contents",
            "config": {"sizes": {k: dict(zip(MEMILORN_NAMES, v)) for k, v in MEMILORN_SIZES.items()}, "block_size": BLOCK, "peaks": pk["source"],
                       "l2": "weights + cache per step larger than L2, no flush"},
            "clocks": sampler.stop(), "sizes": sizes}
    if a.kernels:
        line["kernels"] = memilorn_kernel_points(torch, pk)
    print(json.dumps(line))
    return 0


def luvutar_workload(a) -> int:
    import torch

    from llm_infrence_engine_b200.weights import write_random_model

    pk = peaks()
    sampler = ClockSampler()
    sampler.start()
    sizes = {}
    steps = min(a.steps, 256)
    for size in LUVUTAR_SIZES:
        vocab = LUVUTAR_SIZES[size][-1]
        row = {}
        for name, config in (("luvutar", luvutar_config(size)), ("qwen2", qwen2_like(size))):
            with tempfile.TemporaryDirectory() as tmp:
                folder = write_random_model(config, Path(tmp) / "model", seed=0, store_dtype="bfloat16")
                pt = model_points(folder, vocab, a.batch, a.context or 4096, a.prefill_tokens, steps, max(a.warmup, 3), torch)
            pt["decode_frac_of_copy_peak"] = round(pt["decode_bytes"] / (pt["decode_ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
            row[name] = pt
        sizes[size] = row
    line = {"metric": f"Luvutar beside Qwen2 of equal size: decode (batch {a.batch}, context {a.context or 4096}) and prefill ({a.prefill_tokens} tokens), bf16, random weights",
            "unit": "ms and tokens/s per size", "n_gpus": 1, "impl": "ours", "dtype": "bf16", "steps": steps, "warmup": max(a.warmup, 3),
            "data": "synthetic: random weights (seed 0), uniform random token ids, synthetic cache contents",
            "config": {"sizes": {k: dict(zip(("width", "heads", "kv_heads", "head_dim", "rot_dim", "q_rank", "kv_rank", "window", "ff", "streams", "layers", "vocab"), v))
                                 for k, v in LUVUTAR_SIZES.items()}, "block_size": BLOCK, "peaks": pk["source"],
                       "l2": "weights + cache per step larger than L2, no flush"},
            "clocks": sampler.stop(), "sizes": sizes}
    if a.kernels:
        line["kernels"] = luvutar_kernel_points(torch, pk)
    print(json.dumps(line))
    return 0


def main() -> int:
    global CONTEXT, PREFILL_TOKENS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1024)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", default="0.5b", choices=sorted(SHAPES), help="layer sizes (the default is the one the headline is quoted on)")
    ap.add_argument("--context", type=int, default=0, help="context length of the decode steps (default: the shape's own)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--no-graphs", action="store_true", help="launch every kernel of a decode step from the host instead of replaying a CUDA graph")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"], help="measure one part only (for profiling); the JSON line then lacks the rest")
    ap.add_argument("--workload", default="steps", choices=["steps", "serving", "luvutar", "zepalorn", "mufotar", "memilorn"],
                    help="serving: continuous batching of --requests requests (prompts U[128,2048], outputs U[64,512]) through Engine; "
                         "luvutar, zepalorn: that decoder at two layer sizes beside the Qwen2 decoder of equal size (decode and prefill); "
                         "mufotar: that decoder at two layer sizes beside the Zepalorn decoder of equal size; "
                         "memilorn: that decoder at two layer sizes beside the Mufotar decoder of equal size")
    ap.add_argument("--kernels", action="store_true", help="luvutar, zepalorn, mufotar, memilorn: also time its kernels one by one beside their counterparts")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--token-budget", type=int, default=2048, help="serving: tokens per step (max_num_batched_tokens)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="length of the timed prompt")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm(a)
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    if a.workload == "luvutar":
        return luvutar_workload(a)
    if a.workload == "zepalorn":
        return zepalorn_workload(a)
    if a.workload == "mufotar":
        return mufotar_workload(a)
    if a.workload == "memilorn":
        return memilorn_workload(a)
    PREFILL_TOKENS = a.prefill_tokens
    shape_name, changes, shape_context = SHAPES[a.shape]
    MODEL.update(changes)
    CONTEXT = a.context or shape_context
    a.layers = a.layers or MODEL["num_hidden_layers"]
    a.warmup = max(a.warmup, 3)
    graphs = not a.no_graphs

    import torch

    from llm_infrence_engine_b200.weights import write_random_model

    pk = peaks()
    model = dict(MODEL)
    model["num_hidden_layers"] = a.layers
    with tempfile.TemporaryDirectory() as tmp:
        folder = write_random_model(model, Path(tmp) / "model", seed=0, store_dtype="bfloat16")
        sampler = ClockSampler()
        if a.workload == "serving":
            sampler.start()
            res = serving_point(folder, torch, a.requests, 0, a.token_budget)
            print(json.dumps({"metric": f"output tok/s, continuous batching of {a.requests} requests ({shape_name}, bf16, random weights)",
                              "value": res["output_tok_s"], "unit": "tokens/s", "n_gpus": 1, "impl": "ours", "dtype": "bf16",
                              "config": {"model": shape_name, "layers": a.layers, "layers_of_model": MODEL["num_hidden_layers"],
                                         "prompts": "U[128,2048]", "outputs": "U[64,512]", "seed": 0, "block_size": BLOCK},
                              "clocks": sampler.stop(), "serving": res}))
            return 0
        if a.only == "prefill":  # for profiling the prompt step alone: no decode step runs before it
            pre = prefill_point(folder, torch, graphs=graphs)
            fl = flops_prefill(PREFILL_TOKENS) * a.layers / MODEL["num_hidden_layers"]
            print(json.dumps({"prefill": {"value": round(PREFILL_TOKENS / (pre["ms"] * 1e-3), 1), "tokens": PREFILL_TOKENS,
                                          "ms": round(pre["ms"], 3),
                                          "frac": round(fl / (pre["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
                              "layers": a.layers, "cuda_graphs": graphs}))
            return 0
        main_pt = decode_point(folder, a.batch, a.steps, a.warmup, torch, graphs, sampler)
        clocks = sampler.clocks
        b1 = decode_point(folder, 1, min(a.steps, 256), a.warmup, torch, graphs) if a.only == "all" else None
        b64 = decode_point(folder, 64, min(a.steps, 128), a.warmup, torch, graphs) if a.only == "all" else None
        pre = prefill_point(folder, torch, graphs=graphs) if a.only == "all" else None
        e2e = None if (a.skip_e2e or a.only != "all") else e2e_point(folder, a.batch, min(a.steps, 512), a.warmup, torch, graphs)

    fl = flops_prefill(PREFILL_TOKENS) * a.layers / MODEL["num_hidden_layers"]
    achieved = main_pt["bytes"] / (main_pt["ms"] * 1e-3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {a.batch}, context {CONTEXT} ({shape_name}, bf16, random weights)",
        "value": round(main_pt["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": round(main_pt["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights (seed 0), uniform random token ids, synthetic cache contents",
        "impl": "ours",
        "config": {"model": shape_name, "layers": a.layers, "layers_of_model": MODEL["num_hidden_layers"],
                   "hidden": MODEL["hidden_size"], "heads": MODEL["num_attention_heads"], "kv_heads": MODEL["num_key_value_heads"],
                   "head_dim": MODEL["hidden_size"] // MODEL["num_attention_heads"], "intermediate": MODEL["intermediate_size"],
                   "vocab": MODEL["vocab_size"], "tied": MODEL["tie_word_embeddings"], "global_batch": a.batch, "seq_len": CONTEXT, "block_size": BLOCK, "parallelism": "single GPU",
                   "cuda_graphs": graphs, "l2": "inputs larger than L2 (weights + cache per step >> 126 MB), no flush", "peaks": pk["source"]},
        "clocks": clocks,
        "gpu_launches": main_pt["launches"],
        "prefill": None if pre is None else {
            "value": round(PREFILL_TOKENS / (pre["ms"] * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre["ms"], 3),
            "frac": round(fl / (pre["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": None if b1 is None else {"decode_b1": round(b1["tok_s"], 1), "decode_b64": round(b64["tok_s"], 1)},
        "checked": {"decode_b%d" % a.batch: main_pt["check"], **({} if b1 is None else {"decode_b1": b1["check"], "decode_b64": b64["check"]})},
    }
    if e2e is not None:
        line["e2e"] = {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
