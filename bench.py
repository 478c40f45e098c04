#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama 4 engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--model scout|maverick] [--layers L]
                    [--batch B] [--context C] [--skip-extra]
    python bench.py --case NAME [sizes ...]        # one kernel or one step alone, for ncu

Default: the Scout-layer-sized 16-layer model with seeded random bfloat16 weights, batch 8,
8,192-token contexts. Token ids are uniform over the vocabulary; the caches of the decode
measurements are filled with seeded noise instead of being produced by a prefill (the bytes a
decode step reads are the same). One JSON line is printed:
  value            decoded tokens per second at the default batch, timed on the device
  e2e              the same through hi_b200.LLM (scheduler, sampler, host tokens in and out)
  prefill          one 2,048-token prompt in one step; frac = flops / time / bf16 peak
  roofline         bytes a decode step must read (every weight it uses once + live cache) / time
  points           decode tokens per second at batch 1 and 64, and the two further workloads:
  long_context     the same model at 65,536-token contexts: decoding at batch 1 and 4, and a prompt
                   fed in 4,096-token portions in the same steps as three decoding requests
                   (tokens per second of each portion against its offset, pages in use of the
                   chunked layers step by step: they fall back whenever the prompt passes 8,192)
  maverick         the 4-layer Maverick-sized model (128 experts), batch 64 at 4,096-token contexts:
                   tokens per second, roofline fraction, rows per expert of one step
  cpu_baseline_s   wall time of the plain implementation (tests/plain_llama4.py, whole sequences, no
                   cache, float32 on the CPU) on the two tiny workloads: the timed CPU baseline
The reference (PipeNetwork/hi) runs Llama 4 only through Apple MLX/Metal, so ``--impl
reference`` reports that it is unavailable here.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SCOUT = {
    "architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text",
    "vocab_size": 202048, "hidden_size": 5120, "num_hidden_layers": 16,
    "num_attention_heads": 40, "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 1.0,
                     "original_max_position_embeddings": 8192},
    "attention_chunk_size": 8192, "nope_layer_interval": 4, "use_qk_norm": True,
    "attn_temperature_tuning": True, "floor_scale": 8192, "attn_scale": 0.1,
    "interleave_moe_layer_step": 1, "num_local_experts": 16, "num_experts_per_tok": 1,
    "intermediate_size": 8192, "intermediate_size_mlp": 16384, "tie_word_embeddings": False,
    "max_position_embeddings": 262144,
}
MAVERICK = dict(SCOUT, num_hidden_layers=4, rope_scaling=None, use_qk_norm=False, interleave_moe_layer_step=2,
                num_local_experts=128)
MODELS = {"scout": (SCOUT, 16), "maverick": (MAVERICK, 4)}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
PAGE = 64
DEFAULT_STEPS = 64


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p.get("bf16_tflops_sustained") or p["bf16_tflops"]),
                    "source": "measured"}
        except (ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """SM clock and throttle reasons during the timed regions (read-only NVML queries)."""

    def __init__(self):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake_slowdown": 0x80, "sync_boost": 0x10, "applications_clocks_setting": 0x2}
        while not self._stop.wait(0.2):
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                self.reasons |= {n for n, bit in names.items() if mask & bit}
            except Exception:
                pass

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons)}


def model_bytes_and_flops(model, distinct_by_layer, context):
    """From the built model: bytes of weights and cache one decode step must read for ONE request
    at ``context`` tokens (weights counted once, experts by how many distinct ones the step
    touched), the cache bytes per request, and the matrix flops per token."""
    weight_bytes, kv_bytes, flops = 0, 0, 0
    for i, layer in enumerate(model.layers):
        mix, ff = layer.mixer, layer.feed_forward
        attn = mix.w_qkv.numel() + mix.w_o.numel()
        weight_bytes += 2 * attn + 2 * 2 * model.spec.hidden_size
        flops += 2 * attn
        visible = context
        if mix.window:
            visible = ((context - 1) % mix.window[1]) + 1 if mix.window[0] == "chunk" else min(context, mix.window[1])
        kv_bytes += 2 * 2 * mix.nkv * mix.hd * visible
        if hasattr(ff, "w_gate"):
            expert = 3 * ff.hidden * ff.inter
            shared = ff.shared.w_gate_up.numel() + ff.shared.w_down.numel() if ff.shared else 0
            weight_bytes += 2 * (ff.w_router.numel() + shared + distinct_by_layer.get(i, ff.experts) * expert)
            flops += 2 * (ff.w_router.numel() + shared + ff.top_k * expert)
        else:
            dense = ff.mlp.w_gate_up.numel() + ff.mlp.w_down.numel()
            weight_bytes += 2 * dense
            flops += 2 * dense
    head = 2 * model.spec.vocab_size * model.spec.hidden_size
    return weight_bytes + head, kv_bytes, flops


def attention_flops(model, first, count):
    """Score and value flops of ``count`` new tokens at positions ``first ..`` (each query against
    the keys it may read: all earlier ones, or those of its own chunk)."""
    total = 0
    for layer in model.layers:
        mix = layer.mixer
        if mix.window and mix.window[0] == "chunk":
            c, keys, p, end = mix.window[1], 0, first, first + count
            while p < end:                               # chunk by chunk: a query at p sees p % c + 1 keys
                seg = min(end, (p // c + 1) * c) - p
                keys += seg * (p % c) + seg * (seg + 1) // 2
                p += seg
        else:
            keys = count * first + count * (count + 1) // 2
        total += 4 * mix.nh * mix.hd * keys
    return total


def build_engine(cfg, global_tokens, chunked_tokens, slots):
    """The model with random weights made on the device, pools of the given sizes (tokens), and
    caches filled with seeded noise (decode steps are timed without the prefill that would fill them)."""
    import torch

    from hi_b200.engine.core import Engine

    t0 = time.time()
    engine = Engine.from_config(cfg, seed=0, std=0.02, dtype="bfloat16", kv_page_size=PAGE,
                                kv_cache_tokens=global_tokens, windowed_cache_tokens=chunked_tokens,
                                max_active_requests=slots)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    gen = torch.Generator(device="cuda").manual_seed(1)
    for view in engine.cache.views.values():
        if view.k_pages is not None:
            view.k_pages.normal_(0.0, 1.0, generator=gen)
            view.v_pages.normal_(0.0, 1.0, generator=gen)
    return engine, load_s


def timed_decode(engine, batch, ctx_len, steps, warmup, vocab, cpu_gen, tag="d"):
    """W + K single-token steps of ``batch`` requests whose contexts end at ``ctx_len``; the K
    timed steps lie between two synchronisations, every step has its own event too (median)."""
    import torch

    from hi_b200.engine.core import StepEntry
    from hi_b200.kernels import ops

    total = warmup + steps + 1
    ids = [f"{tag}{batch}-{i}" for i in range(batch)]
    for rid in ids:
        engine.assume_cached(rid, ctx_len - total)
    toks = torch.randint(0, vocab, (total, batch), generator=cpu_gen).tolist()
    # one step with a tap to see which experts a step touches, then the warm-up steps (the first
    # step of a shape is eager, the second captures the CUDA graph of this shape)
    taps = {}
    engine.step([StepEntry(r, [toks[total - 1][i]], [0]) for i, r in enumerate(ids)],
                tap=lambda n, t: taps.__setitem__(n, t.clone()))
    routing = {int(n.split(".")[2]): t.flatten().tolist() for n, t in taps.items() if n.endswith("router_ids")}
    distinct = {layer: len(set(chosen)) for layer, chosen in routing.items()}
    for s in range(warmup):
        engine.step([StepEntry(r, [toks[s][i]], [0]) for i, r in enumerate(ids)])
    torch.cuda.synchronize()
    launches0 = ops.LAUNCHES[0]
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    marks[0].record()
    for k, s in enumerate(range(warmup, total - 1)):
        engine.step([StepEntry(r, [toks[s][i]], [0]) for i, r in enumerate(ids)])
        marks[k + 1].record()
    torch.cuda.synchronize()
    ms = marks[0].elapsed_time(marks[-1]) / steps
    per_step = [marks[k].elapsed_time(marks[k + 1]) for k in range(steps)]
    launches = ops.LAUNCHES[0] - launches0
    for rid in ids:
        engine.finish(rid)
    wb, kv, _ = model_bytes_and_flops(engine.model, distinct, ctx_len)
    return {"ms": ms, "ms_median": statistics.median(per_step), "tok_s": batch * 1000.0 / ms, "launches": launches,
            "distinct": (sum(distinct.values()) / len(distinct) if distinct else 0.0), "bytes": wb + batch * kv,
            "routing": routing}


def release(engine):
    import torch

    engine.model = None
    engine.cache = None
    engine._graphs.clear()
    del engine
    gc.collect()
    torch.cuda.empty_cache()


def long_context_point(engine, cfg, args, pk, vocab, cpu_gen):
    """65,536-token contexts on the same model: decoding at batch 1 and 4, and one request's prompt
    fed in 4,096-token portions in the same steps as three requests that decode."""
    import torch

    from hi_b200.engine.core import StepEntry

    ctx = args.long_context
    out = {"context": ctx}
    steps = max(8, min(args.steps, 32))
    for b in (1, 4):
        r = timed_decode(engine, b, ctx, steps, args.warmup, vocab, cpu_gen, tag="L")
        out[f"decode_b{b}"] = {"value": r["tok_s"], "ms_per_step": r["ms"],
                               "frac": r["bytes"] / (r["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"]}
    portion = args.long_portion
    n_portions = (ctx - portion) // portion
    decoders = [f"Lm{i}" for i in range(3)]
    for rid in decoders:
        engine.assume_cached(rid, ctx - n_portions - 4)
    prompt = torch.randint(0, vocab, (n_portions * portion,), generator=cpu_gen).tolist()
    dec = torch.randint(0, vocab, (n_portions + 1, 3), generator=cpu_gen).tolist()
    chunked = [g for g, spec in enumerate(engine.manager.groups) if spec.window]
    portions, pages = [], []
    # the first portion runs once untimed (warm-up of this step shape), as a request of its own
    engine.step([StepEntry("Lwarm", prompt[:portion], [])] + [StepEntry(r, [dec[n_portions][i]], [0]) for i, r in enumerate(decoders)])
    engine.finish("Lwarm")
    torch.cuda.synchronize()
    for p in range(n_portions):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        entries = [StepEntry("Lp", prompt[p * portion:(p + 1) * portion], [portion - 1] if p == n_portions - 1 else [])]
        entries += [StepEntry(r, [dec[p][i]], [0]) for i, r in enumerate(decoders)]
        start.record()
        engine.step(entries)
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        _, _, fpt = model_bytes_and_flops(engine.model, {}, ctx)
        flops = fpt * (portion + 3) + attention_flops(engine.model, p * portion, portion)
        portions.append({"offset": p * portion, "ms": round(ms, 2), "tokens_per_s": round((portion + 3) * 1000.0 / ms),
                         "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 3)})
        snap = engine.manager.snapshot()["groups"]
        pages.append(sum(snap[g]["used"] for g in chunked))
    for rid in decoders + ["Lp"]:
        engine.finish(rid)
    out["mixed_steps"] = {"portion_tokens": portion, "decoding_requests": 3, "portions": portions,
                          "chunked_pages_in_use_after_each_step": pages, "page_tokens": PAGE}
    # a short portion far into a context: few blocks with long runs of keys, which the layers that
    # see every key share out among several blocks each; timed with that and without
    from hi_b200.kernels import ops

    short = 512
    engine.assume_cached("Ls", ctx - 4 * short)
    toks = torch.randint(0, vocab, (3 * short,), generator=cpu_gen).tolist()
    times = []
    for i, min_tiles in enumerate((None, None, 1 << 30)):       # the first runs untimed
        keep = ops.PREFILL_SPLIT_MIN_TILES
        if min_tiles:
            ops.PREFILL_SPLIT_MIN_TILES = min_tiles
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step([StepEntry("Ls", toks[i * short:(i + 1) * short], [])])
        end.record()
        torch.cuda.synchronize()
        ops.PREFILL_SPLIT_MIN_TILES = keep
        times.append(start.elapsed_time(end))
    engine.finish("Ls")
    out["short_portion"] = {"tokens": short, "offset": ctx - 3 * short, "ms": round(times[1], 2),
                            "ms_one_block_per_query_tile": round(times[2], 2)}
    return out


def maverick_point(args, pk, cpu_gen):
    """The Maverick-sized model (4 layers, two of them with 128 experts), batch 64, 4,096-token contexts."""
    cfg, _full = MODELS["maverick"]
    engine, load_s = build_engine(cfg, 64 * (4096 + PAGE) + 4 * PAGE, 64 * (4096 + 2 * PAGE) + 4 * PAGE, 66)
    r = timed_decode(engine, 64, 4096, max(8, min(args.steps, 32)), args.warmup, cfg["vocab_size"], cpu_gen, tag="M")
    rows = {}
    for layer, chosen in r["routing"].items():
        counts = {}
        for e in chosen:
            counts[e] = counts.get(e, 0) + 1
        hist = {}
        for c in counts.values():
            hist[c] = hist.get(c, 0) + 1
        rows[f"layer{layer}"] = {"experts_with_rows": len(counts), "max_rows": max(counts.values()),
                                 "mean_rows": round(len(chosen) / len(counts), 2),
                                 "experts_by_rows": {str(k): hist[k] for k in sorted(hist)}}
    out = {"value": r["tok_s"], "ms_per_step": r["ms"], "batch": 64, "context": 4096, "layers": cfg["num_hidden_layers"],
           "experts": cfg["num_local_experts"], "bytes_per_step": r["bytes"],
           "frac": r["bytes"] / (r["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], "rows_per_expert": rows,
           "weights_load_s": round(load_s, 1)}
    release(engine)
    return out


def cpu_baseline():
    """Wall time of the plain implementation on the two tiny workloads (4 prompts of 7/19/33/48 tokens
    + 16 generated tokens each on tiny A; 3 prompts of 5/40/70 + 24 on tiny B): greedy generation
    that runs the whole sequence again for every token, float32 on the CPU."""
    import tempfile

    import torch

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_llama4 as plain
    from harness import make_model, random_tokens, read_weights
    from tiny_configs import TINY_A, TINY_B

    out = {}
    threads = torch.get_num_threads()
    for name, cfg, prompts, new in (("tiny_a", TINY_A, (7, 19, 33, 48), 16), ("tiny_b", TINY_B, (5, 40, 70), 24)):
        with tempfile.TemporaryDirectory() as d:
            make_model(d, cfg, seed=11, std=0.08)
            w = read_weights(d)
        t0 = time.perf_counter()
        for i, n in enumerate(prompts):
            toks = random_tokens(cfg, n, seed=50 + i)
            for _ in range(new):
                toks.append(int(plain.forward(cfg, w, toks)[-1].argmax()))
        out[name] = round(time.perf_counter() - t0, 2)
    out["threads"] = threads
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=DEFAULT_STEPS)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="scout", choices=sorted(MODELS))
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--points", default="1,64")
    ap.add_argument("--skip-prefill", action="store_true")
    ap.add_argument("--skip-extra", action="store_true", help="leave out the long-context, Maverick and CPU points")
    ap.add_argument("--long-context", type=int, default=65536)
    ap.add_argument("--long-portion", type=int, default=4096)
    ap.add_argument("--case", nargs="+", default=None, metavar=("NAME", "SIZE"),
                    help="run one kernel or one step alone a few times (for ncu): " + ", ".join(sorted(CASES)))
    args = ap.parse_args(argv)
    if args.case:
        CASES[args.case[0]](*[int(a) for a in args.case[1:]])
        print("ok")
        return 0
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "PipeNetwork/hi runs Llama 4 only through Apple MLX/Metal (crates/hi-mlx, macOS aarch64); "
                          "it is a Rust workspace with no Python package and no Rust toolchain is installed here"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is outside this engine (single-GPU by design)")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch

    import hi_b200
    from hi_b200.engine.core import StepEntry
    from hi_b200.sampling import SamplingParams

    pk = peaks()
    base_cfg, FULL_LAYERS = MODELS[args.model]
    if args.layers is None:
        args.layers = FULL_LAYERS
    cfg = dict(base_cfg, num_hidden_layers=args.layers)
    points = sorted({int(p) for p in args.points.split(",") if p} | {args.batch})
    max_batch = max(points)
    ctx_len = args.context
    extra = not args.skip_extra and args.model == "scout" and args.layers == FULL_LAYERS
    # pools: every request of the largest batch at the context length, the prompt of the prefill point and
    # some slack; rotary layers keep one attention chunk per request (plus the pages being written).
    # The long-context point reuses this engine: four requests of 65,536 tokens, one of them fed in portions
    slack = args.prefill_tokens + 4 * PAGE
    global_tokens = max_batch * (ctx_len + PAGE) + slack
    chunked_tokens = max_batch * (min(ctx_len, cfg["attention_chunk_size"]) + 2 * PAGE) + slack
    if extra:
        global_tokens = max(global_tokens, 4 * (args.long_context + PAGE) + slack)
        chunked_tokens = max(chunked_tokens, 4 * (cfg["attention_chunk_size"] + 2 * PAGE) + args.long_portion + slack)
    engine, load_s = build_engine(cfg, global_tokens, chunked_tokens, max(max_batch, 4) + 2)
    vocab = cfg["vocab_size"]
    cpu_gen = torch.Generator().manual_seed(2)
    sampler = ClockSampler()
    sampler.start()

    results = {b: timed_decode(engine, b, ctx_len, args.steps, args.warmup, vocab, cpu_gen) for b in points}
    main_r = results[args.batch]

    # ---- prefill: one prompt of --prefill-tokens in one step, logits at the last position
    prefill = None
    if not args.skip_prefill:
        T = args.prefill_tokens
        reps = 3
        times = []
        for r in range(reps + 1):
            toks = torch.randint(0, vocab, (T,), generator=cpu_gen).tolist()
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            engine.step([StepEntry("p", toks, [T - 1])])
            end.record()
            torch.cuda.synchronize()
            engine.finish("p")
            if r > 0:
                times.append(start.elapsed_time(end))
        ms = statistics.median(times)
        _, _, fpt = model_bytes_and_flops(engine.model, {}, T)
        nh, hd = cfg["num_attention_heads"], cfg["head_dim"]
        flops = fpt * T + args.layers * 4 * nh * hd * T * T / 2 + 2 * vocab * cfg["hidden_size"]
        prefill = {"value": T * 1000.0 / ms, "tokens": T, "ms": ms, "frac": flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12),
                   "peak_tflops": pk["bf16_tflops"], "peak_source": pk["source"]}

    # ---- end to end through the public entry point: scheduler + sampler, host tokens in and out
    llm = hi_b200.LLM(engine, max_batch_size=args.batch, max_batched_tokens=8192)
    total = args.warmup + args.steps
    reqs = []
    for i in range(args.batch):
        prompt = torch.randint(0, vocab, (ctx_len - total,), generator=cpu_gen).tolist()
        req = llm.add_request(prompt, SamplingParams(max_tokens=total, ignore_eos=True, temperature=0.0), request_id=f"e{i}")
        reqs.append(req)
    # the prompts' keys are taken as cached noise except for their last token
    for req in reqs:
        engine.assume_cached(req.request_id, len(req.prompt) - 1)
        llm.scheduler.assume_running(req, len(req.prompt) - 1)
    for _ in range(args.warmup):
        llm.step()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall = time.perf_counter()
    start.record()
    n_steps = 0
    # tokens the host has read so far, and those of the step that is already running (launched by
    # the last warm-up call; its work lies before the timed region, so its tokens do not count)
    read_before = sum(len(r.output) for r in reqs) + (len(llm._launched.sampling) if llm._launched is not None else 0)
    while any(r.status != "finished" for r in reqs):
        llm.step()
        n_steps += 1
    end.record()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t_wall) * 1000.0
    # tokens that reached the host inside the timed region (a step launched ahead is read one call later)
    e2e_tok_s = (sum(len(r.output) for r in reqs) - read_before) * 1000.0 / max(wall_ms, start.elapsed_time(end))
    h2d = engine.last_step_h2d_bytes          # the packed step inputs (tokens, positions, block tables, ...)
    clocks = sampler.stop()

    line = {
        "metric": f"decode tokens/s (Llama 4 {args.model.capitalize()} layer sizes, bf16)", "value": main_r["tok_s"], "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": main_r["ms"],
        "ms_per_step_median": main_r["ms_median"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0,0.02), uniform random token ids, noise-filled KV cache",
        "config": {"model": f"llama4-{args.model}-layers", "layers": args.layers, "layers_full": FULL_LAYERS,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "experts": cfg["num_local_experts"], "top_k": cfg["num_experts_per_tok"],
                   "expert_inter": cfg["intermediate_size"], "mlp_inter": cfg["intermediate_size_mlp"],
                   "moe_every": cfg.get("interleave_moe_layer_step", 1), "vocab": vocab, "chunk": cfg["attention_chunk_size"],
                   "global_batch": args.batch, "seq_len": ctx_len, "page": PAGE, "parallelism": "single-gpu",
                   "l2": "inputs larger than L2 (each step streams all weights it uses)",
                   "weights_load_s": round(load_s, 1)},
        "clocks": clocks,
        "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch,
                "steps": n_steps},
        "gpu_launches": main_r["launches"],
        "roofline": {"bound": "hbm", "achieved": main_r["bytes"] / (main_r["ms"] * 1e-3) / 1e9, "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": main_r["bytes"] / (main_r["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"],
                     "peak_source": pk["source"], "bytes_per_step": main_r["bytes"],
                     "distinct_experts_per_layer": main_r["distinct"]},
        "points": {f"decode_b{b}": results[b]["tok_s"] for b in points if b != args.batch},
        "points_roofline_frac": {f"decode_b{b}": results[b]["bytes"] / (results[b]["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"]
                                 for b in points},
    }
    if prefill:
        line["prefill"] = prefill
    if extra:
        long_ctx = long_context_point(engine, cfg, args, pk, vocab, cpu_gen)
        line["long_context"] = long_ctx
        line["points"]["decode_b1_ctx65536"] = long_ctx["decode_b1"]["value"]
        line["points"]["decode_b4_ctx65536"] = long_ctx["decode_b4"]["value"]
        llm = None
        release(engine)
        mav = maverick_point(args, pk, cpu_gen)
        line["maverick"] = mav
        line["points"]["maverick_decode_b64_ctx4096"] = mav["value"]
        line["cpu_baseline_s"] = cpu_baseline()
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------- one kernel or one step alone
# Small, fixed cases at the Scout layer's sizes (40 heads, 8 kv heads, head_dim 128; hidden 5120,
# 16 experts of 8192) for `ncu -k regex:<kernel>`: inputs larger than L2, a few GB at most.
DEV = "cuda:0"


def case_decode_attention(batch=8, context=8192, page=64):
    import torch

    from hi_b200.kernels import ops

    nh, nkv, hd = 40, 8, 128
    blocks = -(-context // page)
    g = torch.Generator(device=DEV).manual_seed(0)
    kp = torch.randn(batch * blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    vp = torch.randn(batch * blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    bt = torch.randperm(batch * blocks, device=DEV, generator=g).to(torch.int32).view(batch, blocks).contiguous()
    q = torch.randn(batch, nh, hd, device=DEV, generator=g).to(torch.bfloat16)
    pos = torch.full((batch,), context - 1, dtype=torch.int32, device=DEV)
    sot = torch.arange(batch, dtype=torch.int32, device=DEV)
    for _ in range(3):
        ops.decode_attention(q, kp, vp, bt, sot, pos, 0, 0, hd ** -0.5, context)
    torch.cuda.synchronize()


def case_decode_attention_fused(batch=8, context=8192, page=64):
    """The one-launch form: q/k/v encoding, cache append, attention and merge, on a rotary chunked layer's settings."""
    import torch

    from hi_b200.kernels import ops

    nh, nkv, hd = 40, 8, 128
    blocks = -(-context // page)
    g = torch.Generator(device=DEV).manual_seed(0)
    kp = torch.randn(batch * blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    vp = torch.randn(batch * blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    bt = torch.randperm(batch * blocks, device=DEV, generator=g).to(torch.int32).view(batch, blocks).contiguous()
    qkv = torch.randn(batch, (nh + 2 * nkv) * hd, device=DEV, generator=g).to(torch.bfloat16)
    pos = torch.full((batch,), context - 1, dtype=torch.int32, device=DEV)
    sot = torch.arange(batch, dtype=torch.int32, device=DEV)
    inv = torch.rand(hd // 2, device=DEV, generator=g)
    for _ in range(3):
        ops.decode_attention_fused(qkv, nh, nkv, hd, pos, inv, False, True, 1e-6, None, sot, bt, kp, vp, 8192, 0, hd ** -0.5, context)
    torch.cuda.synchronize()


def _experts(experts, rows):
    import torch

    from hi_b200.kernels import ops

    hidden, inter = 5120, 8192
    g = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn(rows, hidden, device=DEV, generator=g).to(torch.bfloat16)
    wg = (torch.randn(experts, inter, hidden, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    wu = (torch.randn(experts, inter, hidden, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    wd = (torch.randn(experts, hidden, inter, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    ids = torch.randint(0, experts, (rows, 1), device=DEV, generator=g).to(torch.int32)
    scores = torch.rand(rows, 1, device=DEV, generator=g)
    return x, wg, wu, wd, scores, ops.moe_plan(ids, experts)


def case_expert_gemv(batch=8):
    """The weight-streaming expert kernels at decode shape."""
    import torch

    from hi_b200.kernels import ops

    x, wg, wu, wd, scores, plan = _experts(16, batch)
    for _ in range(3):
        act = ops.moe_gate_up(x, plan, 1, wg, wu, scores, True)
        ops.moe_down(act, wd, plan, True)
    torch.cuda.synchronize()


def case_expert_tc(tokens=1024, experts=8):
    """The tcgen05 grouped products at prefill shape: about 128 rows per expert."""
    from hi_b200.kernels import ops

    x, wg, wu, wd, scores, plan = _experts(experts, tokens)
    for _ in range(3):
        act = ops.moe_gate_up_tc(x, plan, 1, wg, wu, scores)
        ops.moe_down_tc(act, wd, plan)
    ops.check_tc_status()


def case_prefill_attention(tokens=2048, cached=0, page=64):
    """One portion of ``tokens`` new tokens behind ``cached`` earlier ones, both prefill kernels."""
    import torch

    from hi_b200.kernels import ops

    nh, nkv, hd = 40, 8, 128
    total = tokens + cached
    blocks = -(-total // page)
    g = torch.Generator(device=DEV).manual_seed(0)
    kp = torch.randn(blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    vp = torch.randn(blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    bt = torch.randperm(blocks, device=DEV, generator=g).to(torch.int32).view(1, blocks).contiguous()
    q = torch.randn(tokens, nh, hd, device=DEV, generator=g).to(torch.bfloat16)
    pos = torch.arange(cached, total, dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, tokens], dtype=torch.int32, device=DEV)
    for _ in range(3):
        if cached == 0:
            ops.prefill_attention(q, kp, vp, bt, cu, pos, 1, tokens, 0, 0, hd ** -0.5)
        ops.prefill_attention_tc(q, kp, vp, bt, cu, pos, 1, tokens, 0, 0, hd ** -0.5)
    ops.check_tc_status()


def _case_engine(layers, tokens, slots):
    from hi_b200.engine.core import Engine

    return Engine.from_config(dict(SCOUT, num_hidden_layers=layers), seed=0, dtype="bfloat16", device=DEV,
                              kv_page_size=PAGE, kv_cache_tokens=tokens, max_active_requests=slots, use_cuda_graphs=False)


def case_decode_step(batch=8, context=8192, layers=2):
    """Three decode steps of ``batch`` requests at ``context`` cached tokens, every kernel launched on its own."""
    import torch

    from hi_b200.engine.core import StepEntry

    eng = _case_engine(layers, batch * (context + 128), batch + 1)
    for i in range(batch):
        eng.assume_cached(i, context - 8)
    g = torch.Generator().manual_seed(0)
    for _ in range(3):
        eng.step([StepEntry(i, [int(torch.randint(0, 202048, (1,), generator=g))], [0]) for i in range(batch)])
    torch.cuda.synchronize()


def case_prefill_step(tokens=2048, layers=2):
    """Three prompts of ``tokens`` tokens, each in one step."""
    import torch

    from hi_b200.engine.core import StepEntry

    eng = _case_engine(layers, tokens + 128, 2)
    g = torch.Generator().manual_seed(0)
    for i in range(3):
        eng.step([StepEntry(i, torch.randint(0, 202048, (tokens,), generator=g).tolist(), [tokens - 1])])
        eng.finish(i)
    torch.cuda.synchronize()


def case_sweep():
    """The hot kernels alone over further sizes, timed with CUDA events (median of five, a buffer
    larger than L2 written between calls), with their fractions of the measured peaks: decode
    attention by batch and context, the expert products by the number of routed tokens (the kernel
    the feed-forward part would pick), prefill attention by portion length and offset. Markdown."""
    import torch

    from hi_b200.kernels import ops
    from hi_b200.parts.attention import AttentionMixer
    from hi_b200.parts.feed_forward import SigmoidRoutedExperts

    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    g = torch.Generator(device=DEV).manual_seed(0)

    def timed(fn):
        fn()
        ts = []
        for _ in range(5):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return sorted(ts)[2]

    nh, nkv, hd, page = 40, 8, 128, 64
    print(f"peaks: {pk['hbm_gbs']:.1f} GB/s copy, {pk['bf16_tflops']:.1f} TFLOP/s bf16 ({pk['source']}); times include the launch\n")
    print("decode attention, 40 heads / 8 kv heads, head_dim 128 (one launch: q/k/v encoding, append, attention, merge; "
          "from 256 (token, kv head) pairs on: qkv_post + attention + merge)\n")
    print("| requests | keys each | us | GB/s of K and V | of the copy peak |\n|---|---|---|---|---|")
    for context in (1024, 8192, 32768, 65536):
        for batch in (1, 2, 4, 8, 16, 32, 64):
            if batch * context > 64 * 8192 * 2:
                continue
            blocks = -(-context // page)
            kp = torch.randn(batch * blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
            vp = torch.randn(batch * blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
            bt = torch.randperm(batch * blocks, device=DEV, generator=g).to(torch.int32).view(batch, blocks).contiguous()
            qkv = torch.randn(batch, (nh + 2 * nkv) * hd, device=DEV, generator=g).to(torch.bfloat16)
            pos = torch.full((batch,), context - 1, dtype=torch.int32, device=DEV)
            sot = torch.arange(batch, dtype=torch.int32, device=DEV)

            def attend():
                o = ops.decode_attention_fused(qkv, nh, nkv, hd, pos, None, False, True, 1e-6, (8192.0, 0.1), sot, bt, kp, vp,
                                               0, 0, hd ** -0.5, context)
                if o is None:
                    q = ops.qkv_post(qkv, nh, nkv, hd, pos, None, False, True, 1e-6, (8192.0, 0.1), sot, bt, kp, vp, page, True)
                    ops.decode_attention(q, kp, vp, bt, sot, pos, 0, 0, hd ** -0.5, context)

            us = timed(attend)
            gbs = batch * context * 2 * nkv * hd * 2 / us / 1e3
            print(f"| {batch} | {context} | {us:.1f} | {gbs:.0f} | {gbs / pk['hbm_gbs']:.2f} |")
            del kp, vp
    x, wg, wu, wd, scores, _plan = _experts(16, 4096)
    print("\nrouted experts, 16 experts top-1, hidden 5120, intermediate 8192: gate/up + SwiGLU, then down\n")
    print("| tokens | experts with rows | kernels | us | GB/s of expert weights | of the copy peak |\n|---|---|---|---|---|---|")
    for n in (1, 2, 4, 8, 10, 12, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096):
        ids = torch.randint(0, 16, (n, 1), device=DEV, generator=g).to(torch.int32)
        plan = ops.moe_plan(ids, 16)
        distinct = int(torch.unique(ids).numel())
        few = n <= SigmoidRoutedExperts.FEW_ROWS

        def experts():
            if few:
                ops.moe_down(ops.moe_gate_up(x[:n], plan, 1, wg, wu, scores[:n], True), wd, plan, True)
            else:
                ops.moe_down_tc(ops.moe_gate_up_tc(x[:n], plan, 1, wg, wu, scores[:n]), wd, plan)

        us = timed(experts)
        gbs = distinct * 3 * 8192 * 5120 * 2 / us / 1e3
        print(f"| {n} | {distinct} | {'weight streaming' if few else 'tcgen05'} | {us:.1f} | {gbs:.0f} | {gbs / pk['hbm_gbs']:.2f} |")
    ops.check_tc_status()
    del x, wg, wu, wd
    print("\nprefill attention (tcgen05), one request, 40 heads / 8 kv heads, head_dim 128, a layer that sees every key\n")
    print("| new tokens | cached before | key shares | us | TFLOP/s | of sustained bf16 |\n|---|---|---|---|---|---|")
    for cached in (0, 8192, 61440):
        for tokens in (128, 256, 512, 1024, 2048, 4096, 8192):
            if cached and tokens > 4096:
                continue
            total = tokens + cached
            blocks = -(-total // page)
            kp = torch.randn(blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
            vp = torch.randn(blocks, nkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
            bt = torch.randperm(blocks, device=DEV, generator=g).to(torch.int32).view(1, blocks).contiguous()
            q = torch.randn(tokens, nh, hd, device=DEV, generator=g).to(torch.bfloat16)
            pos = torch.arange(cached, total, dtype=torch.int32, device=DEV)
            cu = torch.tensor([0, tokens], dtype=torch.int32, device=DEV)
            shares = 1
            if cached >= 2 * tokens:
                shares = ops.prefill_key_splits(nh * -(-tokens // 128), cached // 64, ops.sm_count(DEV))
            us = timed(lambda: ops.prefill_attention_tc(q, kp, vp, bt, cu, pos, 1, tokens, 0, 0, hd ** -0.5, key_splits=shares))
            tf = 4 * nh * hd * (tokens * cached + tokens * (tokens + 1) / 2) / us / 1e6
            print(f"| {tokens} | {cached} | {shares} | {us:.1f} | {tf:.0f} | {tf / pk['bf16_tflops']:.2f} |")
            del kp, vp
    ops.check_tc_status()


# --------------------------------------------------------------------------- Vinurax beside the closest existing model
def _vinurax_config(width, heads, ff, layers, vocab=32000, rank=128):
    """Layers in the order latent, delta, latent reading the first one's cache, latent, ...; head sizes 128."""
    def latent(src=None):
        m = {"heads": heads, "dim": 128, "vdim": 128, "kv_rank": rank, "scale": 128 ** -0.5}
        if src is not None:
            m["kv_from"] = src
        return {"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff}}
    delta = {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": heads, "dim": 128, "vdim": 128, "conv": 4,
                                                "decay_rank": 64, "gate_rank": 64}, "mlp": {"kind": "dense", "ff": ff}}
    order = []
    for i in range(layers):
        order.append(delta if i % 3 == 1 else latent(src=i - 2 if i % 3 == 2 else None))
    return {"architecture": "Vinurax", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": order}


def _dense_llama_config(width, heads, ff, layers, vocab=32000):
    """The closest existing model at equal size: attention with rotary positions over every key, dense SwiGLU
    with the same number of feed-forward parameters (three matrices of 2/3 the inner size)."""
    return {"architectures": ["Llama4ForCausalLM"], "model_type": "llama4_text", "vocab_size": vocab, "hidden_size": width,
            "num_hidden_layers": layers, "num_attention_heads": heads, "num_key_value_heads": max(1, heads // 4),
            "head_dim": 128, "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "rope_scaling": None,
            "attention_chunk_size": 1 << 20, "nope_layer_interval": 0, "use_qk_norm": False,
            "attn_temperature_tuning": False, "interleave_moe_layer_step": 0, "num_local_experts": 1,
            "num_experts_per_tok": 1, "intermediate_size": 8, "intermediate_size_mlp": (2 * ff // 3 + 127) // 128 * 128,
            "tie_word_embeddings": True, "max_position_embeddings": 1 << 20}


def case_vinurax(width=2048, heads=16, ff=8192, layers=6, tokens=2048, batch=8, context=4096):
    """Prefill (one prompt of ``tokens`` in one step) and decode (``batch`` requests at ``context`` cached
    tokens, captured steps) throughput of a Vinurax model with random weights beside a dense Llama-4-shaped
    model of equal width, depth, heads and feed-forward parameters; then the new kernels alone beside their
    like kernels, with bytes moved over the measured copy bandwidth. Markdown on standard output."""
    import torch

    from hi_b200.engine.core import Engine, StepEntry
    from hi_b200.kernels import ops

    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    g = torch.Generator().manual_seed(0)

    def timed(fn, reps=5, flush_l2=True):
        fn()
        ts = []
        for _ in range(reps):
            if flush_l2:
                flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return sorted(ts)[len(ts) // 2]

    print(f"peaks: {pk['hbm_gbs']:.0f} GB/s copy, {pk['bf16_tflops']:.0f} TFLOP/s bf16 ({pk['source']}); "
          f"width {width}, {heads} heads of 128, feed-forward {ff}, {layers} layers, bf16, random weights\n")
    print("| model | prefill tokens/s | ms | decode tokens/s | ms/step | weights GB | launches/decode step |\n|---|---|---|---|---|---|---|")
    for name, cfg in (("Vinurax", _vinurax_config(width, heads, ff, layers)),
                      ("dense Llama-4 shape", _dense_llama_config(width, heads, ff, layers))):
        eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", device=DEV, kv_page_size=PAGE,
                                 kv_cache_tokens=batch * (context + 256) + tokens + 256, max_active_requests=batch + 1)
        vocab = eng.vocab_size
        weights = sum(2 * int(torch.Size(sp.shape).numel()) for sp in eng.model.tensor_specs() if sp.init != "absent") / 1e9
        prompt = torch.randint(0, vocab, (tokens,), generator=g).tolist()

        def prefill():
            eng.step([StepEntry("p", prompt, [tokens - 1])])
            eng.finish("p")
        t_pre = timed(prefill, reps=3)
        for i in range(batch):
            eng.assume_cached(i, context)
        toks = torch.randint(0, vocab, (64, batch), generator=g).tolist()
        turn = [0]

        def decode():
            eng.step([StepEntry(i, [toks[turn[0] % 64][i]], [0]) for i in range(batch)], borrow=True)
            turn[0] += 1
        for _ in range(4):
            decode()
        before = ops.LAUNCHES[0]
        t_dec = timed(decode, reps=9, flush_l2=False)
        launches = (ops.LAUNCHES[0] - before) // 10
        print(f"| {name} | {tokens / t_pre * 1e3:,.0f} | {t_pre:.2f} | {batch / t_dec * 1e3:,.0f} | {t_dec:.3f} | {weights:.2f} | {launches} |")
        del eng
        torch.cuda.empty_cache()

    # ---- kernels alone: bytes that must move over the time, against the copy peak
    bf = torch.bfloat16
    dg = torch.Generator(device=DEV).manual_seed(0)
    rnd = lambda *shape, dt=bf: torch.randn(*shape, device=DEV, generator=dg).to(dt)
    rows = []

    def row(kind, name, ms, nbytes, note=""):
        rows.append(f"| {kind} | {name} | {ms * 1e3:.1f} | {nbytes / 1e6:.1f} | {nbytes / ms / 1e6:,.0f} | "
                    f"{nbytes / ms / 1e6 / pk['hbm_gbs']:.2f} | {note} |")

    for n, what in ((tokens, "prefill"), (batch, "decode")):
        x = rnd(n, width, dt=torch.float32)
        d1, d2, g1, g2 = rnd(n, width), rnd(n, width), rnd(n, width), rnd(n, width)
        depth = layers // 2
        hist = rnd(layers + 1, n, width, dt=torch.float32)
        mix = rnd(depth + 1, dt=torch.float32)
        nrm = [(rnd(1, dt=torch.float32), rnd(width), rnd(width)) for _ in range(2)]
        ms = timed(lambda: ops.gated_depth_dyt(x, [(d1, g1), (d2, g2)], hist, depth, mix, nrm, bf))
        row(what, f"gated sum + average over {depth + 1} results + 2 Dynamic Tanh", ms,
            n * width * (4 + 4 * 2 + 4 * depth + 4 + 4 + 2 * 2), "one launch per layer")
        w = rnd(width)
        ms = timed(lambda: ops.add_rmsnorm(x, d1, w, 1e-5, bf))
        row(what, "like: residual add + RMSNorm", ms, n * width * (4 + 2 + 4 + 2), "two launches per layer")
        up = rnd(n, ff)
        coef = torch.tensor([0.7, 0.9], device=DEV)
        ms = timed(lambda: ops.xielu(up, coef))
        row(what, "xIELU", ms, n * ff * 4)
        gu = rnd(n, 2 * (2 * ff // 3))
        ms = timed(lambda: ops.swiglu(gu))
        row(what, "like: SwiGLU", ms, n * (2 * ff // 3) * 6)
    # the delta rule's kernels: a prompt of `tokens`, then `batch` single tokens
    hd = heads * 128
    C = 3 * hd
    s_len = heads * 128 * 128
    state = torch.zeros(batch + 1, s_len + 3 * C, device=DEV)
    for n, seqs, what in ((tokens, 1, "prefill"), (batch, batch, "decode")):
        proj = rnd(n, C + heads + 128)
        taps = rnd(C, 4, dt=torch.float32)
        a_pre = rnd(n, hd, dt=torch.float32)
        dtb, alog = rnd(hd, dt=torch.float32), rnd(heads, dt=torch.float32)
        cu = torch.arange(0, n + 1, n // seqs, dtype=torch.int32, device=DEV)
        sot = torch.repeat_interleave(torch.arange(seqs, device=DEV), n // seqs).to(torch.int32)
        slots = torch.arange(seqs, dtype=torch.int32, device=DEV)
        ms = timed(lambda: ops.delta_prep(proj, 0, C, taps, state, s_len, a_pre, dtb, alog, cu, sot, slots, heads, heads, 128, 128))
        row(what, "delta rule: convolution, unit q/k, beta, decay", ms, n * (C * 2 + hd * 4 + (C + hd + heads) * 4))
        q, k, v, beta, decay = ops.delta_prep(proj, 0, C, taps, state, s_len, a_pre, dtb, alog, cu, sot, slots, heads, heads, 128, 128)
        ms = timed(lambda: ops.delta_recurrence(q, k, v, beta, decay, state, cu, slots, heads, heads, 128, 128,
                                                single_tokens=seqs == n))
        flops = n * heads * 128 * 128 * 2 * 3
        row(what, "delta rule: recurrence", ms, n * (C + hd + heads + hd) * 4 + 2 * seqs * s_len * 4,
            f"{flops / ms / 1e9:,.1f} TFLOP/s float32 of the recurrence's own arithmetic")
        o, gate, wn = rnd(n, hd, dt=torch.float32), rnd(n, hd), rnd(128)
        ms = timed(lambda: ops.delta_out_norm(o, gate, wn, 1e-5, 128, bf))
        row(what, "delta rule: output norm and gate", ms, n * hd * (4 + 2 + 2))
    # what the mixers do to their projections before attention: the latent into its page, beside q/k/v encoding
    for n, what in ((tokens, "prefill"), (batch, "decode")):
        pages = n // PAGE + 1
        pos = torch.arange(n, dtype=torch.int32, device=DEV)
        sot = torch.zeros(n, dtype=torch.int32, device=DEV)
        table = torch.arange(pages, dtype=torch.int32, device=DEV).view(1, pages)
        lat, wl = rnd(n, 128 + 64), rnd(128)
        pool = torch.zeros(pages, 1, PAGE, 128, dtype=bf, device=DEV)
        ms = timed(lambda: ops.latent_append(lat[:, 64:], wl, 1e-5, pos, sot, table, pool))
        row(what, "latent: RMS norm into its page (latent 128)", ms, n * 128 * 4)
        nkv = max(1, heads // 4)
        qkv = rnd(n, (heads + 2 * nkv) * 128)
        kp, vp = (torch.zeros(pages, nkv, PAGE, 128, dtype=bf, device=DEV) for _ in range(2))
        ms = timed(lambda: ops.qkv_post(qkv, heads, nkv, 128, pos, None, False, False, 1e-6, None, sot, table, kp, vp, PAGE, True))
        row(what, "like: q/k/v encoding and append (no rotation)", ms, n * (heads + 2 * nkv) * 128 * 4)
    print("\n| step | kernel | us | MB that must move | GB/s | of the copy peak | |\n|---|---|---|---|---|---|---|")
    print("\n".join(rows))


def case_vinurax_step(tokens=2048, batch=8, context=4096, width=2048, heads=16, ff=8192, layers=3):
    """One Vinurax prompt step and two decode steps with every kernel launched on its own (no captured graph),
    three layers (latent, delta, latent reading the first one's cache): for a launch list under ncu."""
    import torch

    from hi_b200.engine.core import Engine, StepEntry

    eng = Engine.from_config(_vinurax_config(width, heads, ff, layers), seed=0, dtype="bfloat16", device=DEV, kv_page_size=PAGE,
                             kv_cache_tokens=batch * (context + 256) + tokens + 256, max_active_requests=batch + 1,
                             use_cuda_graphs=False)
    g = torch.Generator().manual_seed(0)
    for rep in range(2):
        eng.step([StepEntry("p", torch.randint(0, eng.vocab_size, (tokens,), generator=g).tolist(), [tokens - 1])])
        eng.finish("p")
    for i in range(batch):
        eng.assume_cached(i, context)
    for _ in range(3):
        eng.step([StepEntry(i, [int(torch.randint(0, eng.vocab_size, (1,), generator=g))], [0]) for i in range(batch)])
    torch.cuda.synchronize()


def case_delta_recurrence(tokens=2048, heads=16, seqs=1):
    """The delta rule's recurrence alone (head sizes 128), each of its register forms twice: for ncu, and timed."""
    import torch

    from hi_b200.kernels import ops

    dg = torch.Generator(device=DEV).manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, device=DEV, generator=dg)
    hd, n = heads * 128, tokens * seqs
    q, k, v = rnd(n, hd) / 128, torch.nn.functional.normalize(rnd(n, heads, 128), dim=-1).view(n, hd).contiguous(), rnd(n, hd)
    beta, decay = torch.rand(n, heads, device=DEV), torch.rand(n, hd, device=DEV) * 0.2 + 0.8
    state = torch.zeros(seqs, heads * 128 * 128, device=DEV)
    cu = torch.arange(0, n + 1, tokens, dtype=torch.int32, device=DEV)
    slots = torch.arange(seqs, dtype=torch.int32, device=DEV)
    for rows in (16, 32):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ops.delta_recurrence(q, k, v, beta, decay, state, cu, slots, heads, heads, 128, 128, rows=rows)
        a.record()
        ops.delta_recurrence(q, k, v, beta, decay, state, cu, slots, heads, heads, 128, 128, rows=rows)
        b.record()
        torch.cuda.synchronize()
        print(f"{rows} rows a lane: {a.elapsed_time(b) * 1e3:.1f} us")

# --------------------------------------------------------------------------- Surinex beside the closest existing models
def _surinex_config(width, heads, ff, layers, vocab=32000, passes=2):
    """Layers in the order gla, pair (sigmoid attention beside the delta rule), latent attention, gla, ...; head sizes
    128 (the latent row is 128 + 64 rotated); the first two layers run ``passes`` times."""
    mlp = {"kind": "dense", "ff": ff}
    gla = {"type": "gla", "mixer": {"heads": heads, "dim": 128, "vdim": 128, "tau": 16.0, "decay_rank": 64}, "mlp": mlp}
    pair = {"type": "parallel", "mlp": mlp, "mixer": {
        "left": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                 "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}},
        "right": {"heads": heads // 2, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "conv": 4}}}
    latent = {"type": "latent_attention", "mlp": mlp, "mixer": {
        "heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 128, "q_rank": width // 2, "scale": 192 ** -0.5,
        "rot": {"base": 500000.0, "dims": 64}}}
    order = [(gla, pair, latent)[i % 3] for i in range(layers)]
    return {"architecture": "Surinex", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "canon": {"taps": 4},
            "layers": order, "loop": {"start": 0, "stop": min(2, layers), "times": passes}}


def case_surinex(width=2048, heads=16, ff=8192, layers=6, tokens=2048, batch=8, context=4096):
    """Prefill (one prompt of ``tokens`` in one step) and decode (``batch`` requests at ``context`` cached tokens,
    captured steps) throughput of a Surinex model with random weights beside Vinurax (the closest existing model:
    latent attention and a delta rule in side-by-side blocks) and a dense Llama-4-shaped model of equal width,
    depth, heads and feed-forward size; then the new kernels alone beside their like kernels, with the bytes that
    must move over the measured copy bandwidth. Markdown on standard output."""
    import torch

    from hi_b200.engine.core import Engine, StepEntry
    from hi_b200.kernels import ops

    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    g = torch.Generator().manual_seed(0)

    def timed(fn, reps=5, flush_l2=True):
        fn()
        ts = []
        for _ in range(reps):
            if flush_l2:
                flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return sorted(ts)[len(ts) // 2]

    print(f"peaks: {pk['hbm_gbs']:.0f} GB/s copy, {pk['bf16_tflops']:.0f} TFLOP/s bf16 ({pk['source']}); "
          f"width {width}, {heads} heads of 128, feed-forward {ff}, {layers} layers, bf16, random weights\n")
    print("| model | layer runs | prefill tokens/s | ms | decode tokens/s | ms/step | weights GB | launches/decode step |\n|---|---|---|---|---|---|---|---|")
    for name, cfg in (("Surinex", _surinex_config(width, heads, ff, layers)), ("Vinurax", _vinurax_config(width, heads, ff, layers)),
                      ("dense Llama-4 shape", _dense_llama_config(width, heads, ff, layers))):
        eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", device=DEV, kv_page_size=PAGE,
                                 kv_cache_tokens=batch * (context + 256) + tokens + 256, max_active_requests=batch + 1)
        vocab = eng.vocab_size
        weights = sum(2 * int(torch.Size(sp.shape).numel()) for sp in eng.model.tensor_specs() if sp.init != "absent") / 1e9
        prompt = torch.randint(0, vocab, (tokens,), generator=g).tolist()

        def prefill():
            eng.step([StepEntry("p", prompt, [tokens - 1])])
            eng.finish("p")
        t_pre = timed(prefill, reps=3)
        for i in range(batch):
            eng.assume_cached(i, context)
        toks = torch.randint(0, vocab, (64, batch), generator=g).tolist()
        turn = [0]

        def decode():
            eng.step([StepEntry(i, [toks[turn[0] % 64][i]], [0]) for i in range(batch)], borrow=True)
            turn[0] += 1
        for _ in range(4):
            decode()
        before = ops.LAUNCHES[0]
        t_dec = timed(decode, reps=9, flush_l2=False)
        launches = (ops.LAUNCHES[0] - before) // 10
        print(f"| {name} | {len(eng.model.spec.schedule)} | {tokens / t_pre * 1e3:,.0f} | {t_pre:.2f} | {batch / t_dec * 1e3:,.0f} | "
              f"{t_dec:.3f} | {weights:.2f} | {launches} |")
        del eng
        torch.cuda.empty_cache()

    # ---- kernels alone: bytes that must move over the time, against the copy peak
    bf, f32 = torch.bfloat16, torch.float32
    dg = torch.Generator(device=DEV).manual_seed(0)
    rnd = lambda *shape, dt=bf: torch.randn(*shape, device=DEV, generator=dg).to(dt)
    rows = []

    def row(kind, name, ms, nbytes, note=""):
        rows.append(f"| {kind} | {name} | {ms * 1e3:.1f} | {nbytes / 1e6:.1f} | {nbytes / ms / 1e6:,.0f} | "
                    f"{nbytes / ms / 1e6 / pk['hbm_gbs']:.2f} | {note} |")

    hd = heads * 128
    nkv = max(1, heads // 4)
    for n, seqs, what in ((tokens, 1, "prefill"), (batch, batch, "decode")):
        cu = torch.arange(0, n + 1, n // seqs, dtype=torch.int32, device=DEV)
        sot = torch.repeat_interleave(torch.arange(seqs, device=DEV), n // seqs).to(torch.int32)
        slots = torch.arange(seqs, dtype=torch.int32, device=DEV)
        # the block: norm, the two convolutions, the sum between passes, the mean of two mixers
        x, h = rnd(n, width, dt=f32), rnd(n, width, dt=f32)
        d1, d2, w = rnd(n, width), rnd(n, width), rnd(width)
        ta, tb = rnd(width, 4, dt=f32), rnd(width, 4, dt=f32)
        cstate = torch.zeros(seqs, 3 * width, device=DEV)
        ms = timed(lambda: ops.add_rmsnorm(x, d1, w, 1e-5, f32, delta2=d2))
        row(what, "residual add of two results + RMSNorm, float32 out", ms, n * width * (4 + 2 + 2 + 4 + 4))
        ms = timed(lambda: ops.add_rmsnorm(x, d1, w, 1e-5, bf))
        row(what, "like: residual add + RMSNorm", ms, n * width * (4 + 2 + 4 + 2), "twice per layer there")
        ms = timed(lambda: ops.canon_conv(h, ta, tb, cstate, cu, sot, slots, bf, single_tokens=seqs == n))
        row(what, "two convolutions of the norm's output (4 taps) + state", ms, n * width * (4 + 2 + 2),
            "one launch" if seqs == n else "two launches")
        emb, vec = rnd(n, width, dt=f32), rnd(width, dt=f32)
        ms = timed(lambda: ops.stream_add(x, d1, d2, emb, vec))
        row(what, "between passes: stream += two results + embedding + vector", ms, n * width * (4 + 2 + 2 + 4 + 4))
        ms = timed(lambda: ops.rmsnorm_mean2(d1, d2, w, w, 1e-5, bf))
        row(what, "mean of two RMS-normed mixer outputs", ms, n * width * 6)
        # gated linear attention
        proj, z, bias = rnd(n, 4 * hd + 64), rnd(n, hd, dt=f32), rnd(hd, dt=f32)
        ms = timed(lambda: ops.gla_prep(proj, 0, hd, 2 * hd, z, bias, 16.0, 128 ** -0.5, hd, hd))
        row(what, "gla: q, k, v to float32, decay", ms, n * hd * (3 * 2 + 4 + 4 * 4))
        q, k, v, decay = ops.gla_prep(proj, 0, hd, 2 * hd, z, bias, 16.0, 128 ** -0.5, hd, hd)
        k = torch.nn.functional.normalize(k.view(n, heads, 128), dim=-1).view(n, hd).contiguous()
        s_len = heads * 128 * 128
        state = torch.zeros(seqs, s_len, device=DEV)
        ms = timed(lambda: ops.delta_recurrence(q, k, v, None, decay, state, cu, slots, heads, heads, 128, 128,
                                                single_tokens=seqs == n, plain=True))
        row(what, "gla: recurrence", ms, n * 4 * hd * 4 + n * hd * 4 + 2 * seqs * s_len * 4,
            f"{n * heads * 128 * 128 * 2 * 2 / ms / 1e9:,.1f} TFLOP/s float32 of its own arithmetic")
        beta = torch.rand(n, heads, device=DEV)
        state.zero_()
        ms = timed(lambda: ops.delta_recurrence(q, k, v, beta, decay, state, cu, slots, heads, heads, 128, 128,
                                                single_tokens=seqs == n))
        row(what, "like: delta rule recurrence", ms, n * 4 * hd * 4 + n * (hd + heads) * 4 + 2 * seqs * s_len * 4,
            f"{n * heads * 128 * 128 * 2 * 3 / ms / 1e9:,.1f} TFLOP/s float32 of its own arithmetic")
        o, wn = rnd(n, hd, dt=f32), rnd(128)
        ms = timed(lambda: ops.delta_out_norm(o, proj[:, 3 * hd: 4 * hd], wn, 1e-5, 128, bf, gate_silu=True))
        row(what, "gla / delta rule: output norm and silu gate", ms, n * hd * (4 + 2 + 2))
    # attention: encoding and the kernels themselves, a prompt of `tokens` and `batch` single tokens at `context`
    for n, seqs, ctx_len, what in ((tokens, 1, tokens, "prefill"), (batch, batch, context, "decode")):
        per = -(-ctx_len // PAGE)
        pages = seqs * per
        pos = (torch.arange(n, device=DEV) if seqs == 1 else torch.full((n,), ctx_len - 1, device=DEV)).to(torch.int32)
        sot = torch.repeat_interleave(torch.arange(seqs, device=DEV), n // seqs).to(torch.int32)
        cu = torch.arange(0, n + 1, n // seqs, dtype=torch.int32, device=DEV)
        table = torch.randperm(pages, device=DEV, generator=dg).to(torch.int32).view(seqs, per).contiguous()
        qkv = rnd(n, (heads + 2 * nkv) * 128)
        kp, vp = rnd(pages, nkv, PAGE, 128), rnd(pages, nkv, PAGE, 128)
        inv = torch.tensor([500000.0 ** (-2.0 * i / 64) for i in range(32)], device=DEV)
        vinv = torch.tensor([500000.0 ** (-2.0 * i / 128) for i in range(64)], device=DEV)
        wq = torch.ones(128, device=DEV)
        ms = timed(lambda: ops.qkv_post(qkv, heads, nkv, 128, pos, inv, True, True, 1e-5, None, sot, table, kp, vp, PAGE, True,
                                        q_norm_weight=wq, k_norm_weight=wq, norm_first=True, norm_dim=128, v_inv_freq=vinv,
                                        v_interleaved=True))
        row(what, "sigmoid attention: weighted q/k norm, rotation, rotated values, append", ms, n * (heads + 2 * nkv) * 128 * 4)
        ms = timed(lambda: ops.qkv_post(qkv, heads, nkv, 128, pos, inv, True, True, 1e-5, None, sot, table, kp, vp, PAGE, True,
                                        q_norm_weight=wq, k_norm_weight=wq, norm_first=True, norm_dim=128))
        row(what, "like: the same without rotated values (Fidatar's encoding)", ms, n * (heads + 2 * nkv) * 128 * 4)
        q = rnd(n, heads, 128)
        pb = rnd(heads, dt=f32) - 4.0
        pairs = n * (n + 1) // 2 if seqs == 1 else n * ctx_len
        kv_bytes = (ctx_len if seqs == 1 else n * ctx_len) * nkv * 128 * 2 * 2 + n * heads * 128 * 4
        ms = timed(lambda: ops.sigmoid_attention(q, kp, vp, table, sot, pos, 0, 0, 128 ** -0.5, pb, ctx_len, v_inv_freq=vinv,
                                                 v_interleaved=True))
        row(what, "sigmoid attention over pages, general kernel (float32, other head sizes)", ms, kv_bytes,
            f"{pairs * heads * 128 * 4 / ms / 1e9:,.1f} TFLOP/s")
        if seqs == 1:
            ms = timed(lambda: ops.sigmoid_prefill_attention_tc(q, kp, vp, table, cu, pos, 1, n, 0, 0, 128 ** -0.5, pb,
                                                                v_inv_freq=vinv, v_interleaved=True))
            row(what, "sigmoid attention, tcgen05 prefill + turn back", ms, kv_bytes, f"{pairs * heads * 128 * 4 / ms / 1e9:,.1f} TFLOP/s")
            ms = timed(lambda: ops.prefill_attention_tc(q, kp, vp, table, cu, pos, 1, n, 0, 0, 128 ** -0.5))
            row(what, "like: softmax attention, tcgen05 prefill", ms, kv_bytes, f"{pairs * heads * 128 * 4 / ms / 1e9:,.1f} TFLOP/s")
        else:
            ms = timed(lambda: ops.sigmoid_decode_attention(q, kp, vp, table, sot, pos, 0, 0, 128 ** -0.5, pb, ctx_len, vinv, True))
            row(what, "sigmoid attention, decode kernel + turn back", ms, kv_bytes)
            ms = timed(lambda: ops.decode_attention(q, kp, vp, table, sot, pos, 0, 0, 128 ** -0.5, ctx_len))
            row(what, "like: softmax attention, decode kernel", ms, kv_bytes)
        # latent rows
        lat, wl = rnd(n, 128 + 64 + 32), rnd(128)
        pool = torch.zeros(pages, 1, PAGE, 192, dtype=bf, device=DEV)
        ms = timed(lambda: ops.latent_append(lat[:, 32:], wl, 1e-5, pos, sot, table, pool, inv_freq=inv))
        row(what, "latent: RMS norm + rotated key part into its page (128 + 64)", ms, n * 192 * 4)
        pool2 = torch.zeros(pages, 1, PAGE, 128, dtype=bf, device=DEV)
        ms = timed(lambda: ops.latent_append(lat[:, 32: 160], wl, 1e-5, pos, sot, table, pool2))
        row(what, "like: latent RMS norm into its page (128)", ms, n * 128 * 4)
        ql = rnd(n, heads, 192)
        lat_bytes = (ctx_len if seqs == 1 else n * ctx_len) * 192 * 2 + n * heads * 192 * 4
        if seqs == 1:
            ms = timed(lambda: ops.prefill_attention_tc(ql, pool, pool, table, cu, pos, 1, n, 0, 0, 192 ** -0.5))
        else:
            ms = timed(lambda: ops.decode_attention(ql[:, :16].contiguous(), pool, pool, table, sot, pos, 0, 0, 192 ** -0.5, ctx_len))
            ms *= -(-heads // 16)                            # sixteen heads of the one shared row a call
        row(what, "latent attention over rows of 192 (tensor-core kernel)", ms, lat_bytes, f"{pairs * heads * 192 * 4 / ms / 1e9:,.1f} TFLOP/s")
        ql2 = rnd(n, heads, 128)
        if seqs == 1:
            ms = timed(lambda: ops.prefill_attention_tc(ql2, pool2, pool2, table, cu, pos, 1, n, 0, 0, 128 ** -0.5))
        else:
            ms = timed(lambda: ops.decode_attention(ql2, pool2, pool2, table, sot, pos, 0, 0, 128 ** -0.5, ctx_len))
        row(what, "like: Vinurax's latent attention over rows of 128 (tensor-core kernel)", ms,
            (ctx_len if seqs == 1 else n * ctx_len) * 128 * 2 + n * heads * 128 * 4, f"{pairs * heads * 128 * 4 / ms / 1e9:,.1f} TFLOP/s")
    ops.check_tc_status()
    print("\n| step | kernel | us | MB that must move | GB/s | of the copy peak | |\n|---|---|---|---|---|---|---|")
    print("\n".join(rows))


def case_surinex_step(tokens=2048, batch=8, context=4096, width=2048, heads=16, ff=8192, layers=3):
    """One Surinex prompt step and two decode steps with every kernel launched on its own (no captured graph),
    three layers (gla, pair, latent attention; the first two run twice): for a launch list under ncu."""
    import torch

    from hi_b200.engine.core import Engine, StepEntry

    eng = Engine.from_config(_surinex_config(width, heads, ff, layers), seed=0, dtype="bfloat16", device=DEV, kv_page_size=PAGE,
                             kv_cache_tokens=batch * (context + 256) + tokens + 256, max_active_requests=batch + 1,
                             use_cuda_graphs=False)
    g = torch.Generator().manual_seed(0)
    for rep in range(2):
        eng.step([StepEntry("p", torch.randint(0, eng.vocab_size, (tokens,), generator=g).tolist(), [tokens - 1])])
        eng.finish("p")
    for i in range(batch):
        eng.assume_cached(i, context)
    for _ in range(3):
        eng.step([StepEntry(i, [int(torch.randint(0, eng.vocab_size, (1,), generator=g))], [0]) for i in range(batch)])
    torch.cuda.synchronize()


# --------------------------------------------------------------------------- Bezasun beside the closest existing models
def _bezasun_config(width, heads, ff, layers, vocab=32000, streams=4, window=4096):
    """Layers in the order latent attention (heads of 128 + 64 rotated over a latent of 128, a window), Mamba-2 (twice
    the width in heads of 128 over 128 state channels), attention (heads of 128, a quarter as many key heads, capped
    scores, distance bias, learned sink); every layer with 8 experts of half the dense size, 2 a token, and a shared
    expert of the same size; ``streams`` copies of the residual stream."""
    moe = {"kind": "moe", "expert": {"ff": ff // 2}, "router": {"experts": 8, "top": 2}, "shared": {"ff": ff // 2}}
    latent = {"type": "latent_attention", "mlp": moe, "mixer": {
        "heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 128, "q_rank": width // 2, "scale": 192 ** -0.5,
        "mask": {"size": window},
        "rot": {"base": 10000.0, "dims": 64, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    mamba = {"type": "mamba2", "mlp": moe, "mixer": {"heads": 2 * width // 128, "vdim": 128, "state": 128, "groups": 4,
                                                      "conv": 4, "norm_groups": 4}}
    att = {"type": "attention", "mlp": moe, "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128,
                                                      "scale": 128 ** -0.5, "softcap": 30.0, "q_temp": {"coef": 0.5, "every": 256}}}
    order = [(latent, mamba, att)[i % 3] for i in range(layers)]
    return {"architecture": "Bezasun", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
            "residual_mult": 0.7, "logit_scale": 2.0, "streams": streams, "layers": order}


def case_bezasun(width=2048, heads=16, ff=8192, layers=6, tokens=2048, batch=8, context=4096):
    """Prefill (one prompt of ``tokens`` in one step) and decode (``batch`` requests at ``context`` cached tokens,
    captured steps) throughput of a Bezasun model with random weights beside Fidatar (the closest existing model:
    attention with a sink in turn with a matrix memory, routed experts) and a dense Llama-4-shaped model of equal
    width, depth and heads; then the new and the extended kernels alone beside their like kernels, with the bytes
    that must move over the measured copy bandwidth. Markdown on standard output."""
    import torch

    from hi_b200.engine.core import Engine, StepEntry
    from hi_b200.kernels import ops

    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    g = torch.Generator().manual_seed(0)

    def timed(fn, reps=5, flush_l2=True):
        fn()
        ts = []
        for _ in range(reps):
            if flush_l2:
                flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return sorted(ts)[len(ts) // 2]

    print(f"peaks: {pk['hbm_gbs']:.0f} GB/s copy, {pk['bf16_tflops']:.0f} TFLOP/s bf16 ({pk['source']}); "
          f"width {width}, {heads} heads of 128, feed-forward {ff}, {layers} layers, bf16, random weights\n")
    print("| model | prefill tokens/s | ms | decode tokens/s | ms/step | weights GB | launches/decode step |\n|---|---|---|---|---|---|---|")
    for name, cfg in (("Bezasun", _bezasun_config(width, heads, ff, layers)), ("Fidatar", _fidatar_config(width, heads, ff, layers)),
                      ("dense Llama-4 shape", _dense_llama_config(width, heads, ff, layers))):
        eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", device=DEV, kv_page_size=PAGE,
                                 kv_cache_tokens=batch * (context + 256) + tokens + 256, max_active_requests=batch + 1)
        vocab = eng.vocab_size
        weights = sum(2 * int(torch.Size(sp.shape).numel()) for sp in eng.model.tensor_specs() if sp.init != "absent") / 1e9
        prompt = torch.randint(0, vocab, (tokens,), generator=g).tolist()

        def prefill():
            eng.step([StepEntry("p", prompt, [tokens - 1])])
            eng.finish("p")
        t_pre = timed(prefill, reps=3)
        for i in range(batch):
            eng.assume_cached(i, context)
        toks = torch.randint(0, vocab, (64, batch), generator=g).tolist()
        turn = [0]

        def decode():
            eng.step([StepEntry(i, [toks[turn[0] % 64][i]], [0]) for i in range(batch)], borrow=True)
            turn[0] += 1
        for _ in range(4):
            decode()
        before = ops.LAUNCHES[0]
        t_dec = timed(decode, reps=9, flush_l2=False)
        launches = (ops.LAUNCHES[0] - before) // 10
        print(f"| {name} | {tokens / t_pre * 1e3:,.0f} | {t_pre:.2f} | {batch / t_dec * 1e3:,.0f} | {t_dec:.3f} | {weights:.2f} | {launches} |")
        del eng
        torch.cuda.empty_cache()

    # ---- kernels alone: bytes that must move over the time, against the copy peak
    bf, f32 = torch.bfloat16, torch.float32
    dg = torch.Generator(device=DEV).manual_seed(0)
    rnd = lambda *shape, dt=bf: torch.randn(*shape, device=DEV, generator=dg).to(dt)
    rows = []

    def row(kind, name, ms, nbytes, note=""):
        rows.append(f"| {kind} | {name} | {ms * 1e3:.1f} | {nbytes / 1e6:.1f} | {nbytes / ms / 1e6:,.0f} | "
                    f"{nbytes / ms / 1e6 / pk['hbm_gbs']:.2f} | {note} |")

    copies = 4
    m_heads, m_state, m_groups, m_taps = 2 * width // 128, 128, 4, 4
    inner, gn = m_heads * 128, m_groups * m_state
    channels = inner + 2 * gn
    nkv = max(1, heads // 4)
    for n, seqs, what in ((tokens, 1, "prefill"), (batch, batch, "decode")):
        cu = torch.arange(0, n + 1, n // seqs, dtype=torch.int32, device=DEV)
        sot = torch.repeat_interleave(torch.arange(seqs, device=DEV), n // seqs).to(torch.int32)
        slots = torch.arange(seqs, dtype=torch.int32, device=DEV)
        # the boundary of a stream of copies beside the residual add + RMSNorm
        streams, x = rnd(n, copies, width, dt=f32), rnd(n, width, dt=f32)
        d1, w32, w = rnd(n, width), rnd(width, dt=f32), rnd(width)
        mix, oc, ic = rnd(copies, copies, dt=f32), rnd(copies, dt=f32), rnd(copies, dt=f32)
        ms = timed(lambda: ops.hyper_step(streams, w32, 1e-5, bf, delta=d1, mix=mix, out_coef=oc, mult=0.7, in_coef=ic))
        row(what, f"boundary of {copies} copies: update, weighted sum, RMSNorm", ms, n * width * (copies * 8 + 2 + 2))
        routed, slot = rnd(2 * n, width, dt=f32), torch.randperm(2 * n, device=DEV, generator=dg).to(torch.int32)
        rw = torch.rand(2 * n, device=DEV, generator=dg)
        ms = timed(lambda: ops.hyper_step(streams, w32, 1e-5, bf, delta=d1, routed=routed, slot_of_entry=slot, top_k=2,
                                          routed_weight=rw, mix=mix, out_coef=oc, mult=0.7, in_coef=ic, also_f32=True))
        row(what, "the same with two routed rows a token and a float32 copy of the output", ms, n * width * (copies * 8 + 2 + 8 + 2 + 4))
        ms = timed(lambda: ops.add_rmsnorm(x, d1, w, 1e-5, bf))
        row(what, "like: residual add + RMSNorm (one stream)", ms, n * width * (4 + 2 + 4 + 2))
        ms = timed(lambda: ops.add_rmsnorm(x, d1, w, 1e-5, bf, None, True, routed, slot, 2, rw))
        row(what, "like: the same with two routed rows and a float32 copy", ms, n * width * (4 + 2 + 8 + 4 + 2 + 4))
        # Mamba-2 around its recurrence
        proj = rnd(n, inner + channels + m_heads)
        taps, cb = rnd(channels, m_taps, dt=f32), rnd(channels, dt=f32)
        s_len = m_heads * m_state * 128
        state = torch.zeros(seqs, s_len + (m_taps - 1) * channels, device=DEV)
        dtb, alog, dsk = rnd(m_heads, dt=f32), rnd(m_heads, dt=f32) - 2.0, rnd(m_heads, dt=f32)
        prep = lambda: ops.mamba2_prep(proj, inner, inner + channels, taps, cb, state, s_len, dtb, alog, cu, sot, slots,
                                       m_heads, m_groups, m_state, 128)
        ms = timed(prep)
        row(what, "mamba2: convolution, silu, dt, decay; x, dt x, B, C to float32", ms,
            n * (channels * 2 + (2 * inner + 2 * gn + m_heads * m_state) * 4))
        xx, v, k, q, decay = prep()
        ms = timed(lambda: ops.delta_conv_update(proj, inner, channels, m_taps, state, s_len, cu, slots))
        row(what, "mamba2: the convolution's rows of the state", ms, seqs * (m_taps - 1) * channels * 8)
        ms = timed(lambda: ops.delta_recurrence(q, k, v, None, decay, state, cu, slots, m_heads, m_groups, m_state, 128,
                                                single_tokens=seqs == n, plain=True))
        row(what, f"mamba2: recurrence ({m_heads} heads of 128 x 128)", ms, n * (2 * inner + 2 * gn + m_heads * m_state) * 4 + 2 * seqs * s_len * 4,
            f"{n * m_heads * 128 * 128 * 2 * 2 / ms / 1e9:,.1f} TFLOP/s float32 of its own arithmetic")
        hd16 = heads * 128
        q2, k2, v2, dec2 = rnd(n, hd16, dt=f32), rnd(n, hd16, dt=f32), rnd(n, hd16, dt=f32), torch.rand(n, hd16, device=DEV)
        st2 = torch.zeros(seqs, heads * 128 * 128, device=DEV)
        beta = torch.rand(n, heads, device=DEV)
        ms = timed(lambda: ops.delta_recurrence(q2, k2, v2, beta, dec2, st2, cu, slots, heads, heads, 128, 128, single_tokens=seqs == n))
        row(what, f"like: delta rule recurrence ({heads} heads of 128 x 128)", ms, n * 4 * hd16 * 4 + 2 * seqs * heads * 128 * 128 * 4,
            f"{n * heads * 128 * 128 * 2 * 3 / ms / 1e9:,.1f} TFLOP/s float32 of its own arithmetic")
        o, wn = rnd(n, inner, dt=f32), rnd(inner)
        ms = timed(lambda: ops.mamba2_out(o, xx, proj[:, :inner], dsk, wn, 1e-5, m_heads, 128, 4, bf))
        row(what, "mamba2: skip, silu gate, grouped RMS norm", ms, n * inner * (4 + 4 + 2 + 2))
        o2, wn2 = rnd(n, hd16, dt=f32), rnd(128)
        ms = timed(lambda: ops.delta_out_norm(o2, proj[:, :hd16], wn2, 1e-5, 128, bf, gate_silu=True))
        row(what, "like: delta rule output norm and silu gate", ms, n * hd16 * (4 + 2 + 2))
    # attention with reshaped scores beside the plain softmax, a prompt of `tokens` and `batch` single tokens at `context`
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], device=DEV)
    sinks = torch.randn(heads, device=DEV, generator=dg)
    for n, seqs, ctx_len, what in ((tokens, 1, tokens, "prefill"), (batch, batch, context, "decode")):
        per = -(-ctx_len // PAGE)
        pages = seqs * per
        pos = (torch.arange(n, device=DEV) if seqs == 1 else torch.full((n,), ctx_len - 1, device=DEV)).to(torch.int32)
        sot = torch.repeat_interleave(torch.arange(seqs, device=DEV), n // seqs).to(torch.int32)
        cu = torch.arange(0, n + 1, n // seqs, dtype=torch.int32, device=DEV)
        table = torch.randperm(pages, device=DEV, generator=dg).to(torch.int32).view(seqs, per).contiguous()
        kp, vp = rnd(pages, nkv, PAGE, 128), rnd(pages, nkv, PAGE, 128)
        q = rnd(n, heads, 128)
        pairs = n * (n + 1) // 2 if seqs == 1 else n * ctx_len
        kv_bytes = (ctx_len if seqs == 1 else n * ctx_len) * nkv * 128 * 2 * 2 + n * heads * 128 * 4
        kw = {"softcap": 30.0, "slopes": slopes, "sink_values": sinks}
        if seqs == 1:
            ms = timed(lambda: ops.prefill_attention_tc(q, kp, vp, table, cu, pos, 1, n, 0, 0, 128 ** -0.5, **kw))
            row(what, "attention with cap, distance bias, learned sink: tcgen05 prefill", ms, kv_bytes, f"{pairs * heads * 128 * 4 / ms / 1e9:,.1f} TFLOP/s")
            ms = timed(lambda: ops.prefill_attention_tc(q, kp, vp, table, cu, pos, 1, n, 0, 0, 128 ** -0.5, sink=True))
            row(what, "like: softmax with a sink of score 0, tcgen05 prefill", ms, kv_bytes, f"{pairs * heads * 128 * 4 / ms / 1e9:,.1f} TFLOP/s")
        else:
            ms = timed(lambda: ops.decode_attention(q, kp, vp, table, sot, pos, 0, 0, 128 ** -0.5, ctx_len, **kw))
            row(what, "attention with cap, distance bias, learned sink: decode kernel (cp.async tiles)", ms, kv_bytes)
            ms = timed(lambda: ops.decode_attention(q, kp, vp, table, sot, pos, 0, 0, 128 ** -0.5, ctx_len, sink=True))
            row(what, "like: softmax with a sink of score 0, decode kernel (TMA tiles)", ms, kv_bytes)
        # latent rows with ramped frequencies and interleaved pairs
        inv = torch.tensor([10000.0 ** (-2.0 * i / 64) for i in range(32)], device=DEV)
        lat, wl = rnd(n, 128 + 64), rnd(128)
        pool = torch.zeros(pages, 1, PAGE, 192, dtype=bf, device=DEV)
        ms = timed(lambda: ops.latent_append(lat, wl, 1e-5, pos, sot, table, pool, inv_freq=inv, interleaved=True, rot_mul=1.2))
        row(what, "latent: RMS norm + rotated key part (interleaved, factor) into its page", ms, n * 192 * 4)
        ms = timed(lambda: ops.latent_append(lat, wl, 1e-5, pos, sot, table, pool, inv_freq=inv))
        row(what, "like: the same in halves without a factor", ms, n * 192 * 4)
    ops.check_tc_status()
    print("\n| step | kernel | us | MB that must move | GB/s | of the copy peak | |\n|---|---|---|---|---|---|---|")
    print("\n".join(rows))


def case_bezasun_step(tokens=2048, batch=8, context=4096, width=2048, heads=16, ff=8192, layers=3):
    """One Bezasun prompt step and two decode steps with every kernel launched on its own (no captured graph), three
    layers (latent attention, Mamba-2, attention): for a launch list under ncu."""
    import torch

    from hi_b200.engine.core import Engine, StepEntry

    eng = Engine.from_config(_bezasun_config(width, heads, ff, layers), seed=0, dtype="bfloat16", device=DEV, kv_page_size=PAGE,
                             kv_cache_tokens=batch * (context + 256) + tokens + 256, max_active_requests=batch + 1,
                             use_cuda_graphs=False)
    g = torch.Generator().manual_seed(0)
    for rep in range(2):
        eng.step([StepEntry("p", torch.randint(0, eng.vocab_size, (tokens,), generator=g).tolist(), [tokens - 1])])
        eng.finish("p")
    for i in range(batch):
        eng.assume_cached(i, context)
    for _ in range(3):
        eng.step([StepEntry(i, [int(torch.randint(0, eng.vocab_size, (1,), generator=g))], [0]) for i in range(batch)])
    torch.cuda.synchronize()


def case_bezasun_attention(tokens=2048, heads=16, reshaped=1):
    """The tcgen05 prefill attention alone on one prompt of ``tokens``, with capped scores, a distance bias and a learned
    sink (``reshaped`` = 1) or as the plain softmax with a sink of score 0: three launches, for a capture under ncu."""
    import torch

    from hi_b200.kernels import ops

    bf = torch.bfloat16
    dg = torch.Generator(device=DEV).manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, device=DEV, generator=dg).to(bf)
    nkv, per = max(1, heads // 4), -(-tokens // PAGE)
    pos = torch.arange(tokens, device=DEV).to(torch.int32)
    cu = torch.tensor([0, tokens], dtype=torch.int32, device=DEV)
    table = torch.randperm(per, device=DEV, generator=dg).to(torch.int32).view(1, per).contiguous()
    kp, vp, q = rnd(per, nkv, PAGE, 128), rnd(per, nkv, PAGE, 128), rnd(tokens, heads, 128)
    kw = {"sink": True}
    if reshaped:
        kw = {"softcap": 30.0, "slopes": torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], device=DEV),
              "sink_values": torch.randn(heads, device=DEV, generator=dg)}
    for _ in range(3):
        ops.prefill_attention_tc(q, kp, vp, table, cu, pos, 1, tokens, 0, 0, 128 ** -0.5, **kw)
    torch.cuda.synchronize()
    ops.check_tc_status()


# --------------------------------------------------------------------------- Fidatar beside the closest existing models
def _fidatar_config(width, heads, ff, layers, vocab=32000, chunk=8192):
    """Layers in turn attention (heads of 128, a quarter as many key heads, chunks of 8,192, half of a head
    rotating) and matrix memory (heads of 128); the feed-forward is dense on every third layer and otherwise 8
    experts in 4 groups of which 2 stay open, 2 experts a token, each half the dense size."""
    att = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
           "mask": {"size": chunk}, "rot": {"base": 1e6, "dims": 64, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    mem = {"heads": heads, "dim": 128, "vdim": 128, "gate_cap": 15.0}
    moe = {"kind": "moe", "expert": {"ff": ff // 2}, "router": {"experts": 8, "top": 2, "scale": 1.5, "groups": {"count": 4, "keep": 2}}}
    order = [{"type": "attention" if i % 2 == 0 else "mlstm", "mixer": att if i % 2 == 0 else mem,
              "mlp": {"kind": "dense", "ff": ff} if i % 3 == 0 else moe} for i in range(layers)]
    return {"architecture": "Fidatar", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 8.0},
            "postln_alpha": 2.0, "logit_softcap": 30.0, "layers": order}


def case_fidatar(width=2048, heads=16, ff=8192, layers=6, tokens=2048, batch=8, context=4096):
    """Prefill (one prompt of ``tokens`` in one step) and decode (``batch`` requests at ``context`` cached tokens,
    captured steps) throughput of a Fidatar model with random weights beside Vinurax (the closest existing
    model: attention layers in turn with recurrent ones) and a dense Llama-4-shaped model of equal width, depth
    and heads; then the new and the extended kernels alone beside their like kernels, with the bytes that must
    move over the measured copy bandwidth. Markdown on standard output."""
    import torch

    from hi_b200.engine.core import Engine, StepEntry
    from hi_b200.kernels import ops
    from hi_b200.parts.basic import yarn_inverse_frequencies

    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    g = torch.Generator().manual_seed(0)

    def timed(fn, reps=5, flush_l2=True):
        fn()
        ts = []
        for _ in range(reps):
            if flush_l2:
                flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return sorted(ts)[len(ts) // 2]

    print(f"peaks: {pk['hbm_gbs']:.0f} GB/s copy, {pk['bf16_tflops']:.0f} TFLOP/s bf16 ({pk['source']}); "
          f"width {width}, {heads} heads of 128, feed-forward {ff}, {layers} layers, bf16, random weights\n")
    print("| model | prefill tokens/s | ms | decode tokens/s | ms/step | weights GB | launches/decode step |\n|---|---|---|---|---|---|---|")
    for name, cfg in (("Fidatar", _fidatar_config(width, heads, ff, layers)), ("Vinurax", _vinurax_config(width, heads, ff, layers)),
                      ("dense Llama-4 shape", _dense_llama_config(width, heads, ff, layers))):
        eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", device=DEV, kv_page_size=PAGE,
                                 kv_cache_tokens=batch * (context + 256) + tokens + 256, max_active_requests=batch + 1)
        vocab = eng.vocab_size
        weights = sum(2 * int(torch.Size(sp.shape).numel()) for sp in eng.model.tensor_specs() if sp.init != "absent") / 1e9
        prompt = torch.randint(0, vocab, (tokens,), generator=g).tolist()

        def prefill():
            eng.step([StepEntry("p", prompt, [tokens - 1])])
            eng.finish("p")
        t_pre = timed(prefill, reps=3)
        for i in range(batch):
            eng.assume_cached(i, context)
        toks = torch.randint(0, vocab, (64, batch), generator=g).tolist()
        turn = [0]

        def decode():
            eng.step([StepEntry(i, [toks[turn[0] % 64][i]], [0]) for i in range(batch)], borrow=True)
            turn[0] += 1
        for _ in range(4):
            decode()
        before = ops.LAUNCHES[0]
        t_dec = timed(decode, reps=9, flush_l2=False)
        launches = (ops.LAUNCHES[0] - before) // 10
        print(f"| {name} | {tokens / t_pre * 1e3:,.0f} | {t_pre:.2f} | {batch / t_dec * 1e3:,.0f} | {t_dec:.3f} | {weights:.2f} | {launches} |")
        del eng
        torch.cuda.empty_cache()
    ops.check_tc_status()

    # ---- kernels alone: bytes that must move over the time, against the copy peak
    bf = torch.bfloat16
    dg = torch.Generator(device=DEV).manual_seed(0)
    rnd = lambda *shape, dt=bf: torch.randn(*shape, device=DEV, generator=dg).to(dt)
    rows = []

    def row(kind, name, ms, nbytes, note=""):
        rows.append(f"| {kind} | {name} | {ms * 1e3:.1f} | {nbytes / 1e6:.1f} | {nbytes / ms / 1e6:,.0f} | "
                    f"{nbytes / ms / 1e6 / pk['hbm_gbs']:.2f} | {note} |")

    hd, nkv = heads * 128, max(1, heads // 4)
    inv, mag = yarn_inverse_frequencies(64, 1e6, {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0})
    inv = torch.from_numpy(inv).to(DEV)
    plain_inv = torch.from_numpy(yarn_inverse_frequencies(128, 1e6, None)[0]).to(DEV)
    for n, seqs, what in ((tokens, 1, "prefill"), (batch, batch, "decode")):
        x, d1, w = rnd(n, width, dt=torch.float32), rnd(n, width), rnd(width)
        ms = timed(lambda: ops.add_rmsnorm(x, d1, w, 1e-6, bf, x_scale=2.0, post=True))
        row(what, "post-norm boundary: scaled stream + delta, RMS norm, stream and its rounding written", ms, n * width * (4 + 2 + 4 + 2))
        ms = timed(lambda: ops.add_rmsnorm(x, d1, w, 1e-6, bf))
        row(what, "like: residual add + RMSNorm (pre-norm)", ms, n * width * (4 + 2 + 4 + 2), "the same kernel")
        up = rnd(n, ff)
        ms = timed(lambda: ops.relu2(up))
        row(what, "squared relu", ms, n * ff * 4)
        gu = rnd(n, 2 * (2 * ff // 3))
        ms = timed(lambda: ops.swiglu(gu))
        row(what, "like: SwiGLU", ms, n * (2 * ff // 3) * 6)
        # encoding of q, k, v and the append
        pages = n // PAGE + 1
        pos = torch.arange(n, dtype=torch.int32, device=DEV)
        sot = torch.zeros(n, dtype=torch.int32, device=DEV)
        table = torch.arange(pages, dtype=torch.int32, device=DEV).view(1, pages)
        qkv = rnd(n, (heads + 2 * nkv) * 128)
        kp, vp = (torch.zeros(pages, nkv, PAGE, 128, dtype=bf, device=DEV) for _ in range(2))
        wq, wk = rnd(128, dt=torch.float32), rnd(128, dt=torch.float32)
        ms = timed(lambda: ops.qkv_post(qkv, heads, nkv, 128, pos, inv, False, True, 1e-6, None, sot, table, kp, vp, PAGE, True,
                                        q_norm_weight=wq, k_norm_weight=wk, norm_first=True, norm_dim=128, rot_mul=mag))
        row(what, "q/k/v encoding: weighted norm, then 64 of 128 dims rotate with a magnitude factor; append", ms,
            n * (heads + 2 * nkv) * 128 * 4)
        ms = timed(lambda: ops.qkv_post(qkv, heads, nkv, 128, pos, plain_inv, False, True, 1e-6, None, sot, table, kp, vp, PAGE, True))
        row(what, "like: q/k/v encoding (rotation of all dims, then the weightless norm) and append", ms, n * (heads + 2 * nkv) * 128 * 4)
        # the matrix memory beside the delta rule
        state = torch.zeros(seqs, ops.mlstm_state_floats(heads, 128, 128), device=DEV)
        proj = rnd(n, 4 * hd)
        z = rnd(n, 2 * heads, dt=torch.float32)
        bi, bfg = rnd(heads, dt=torch.float32), rnd(heads, dt=torch.float32) + 3
        cu = torch.arange(0, n + 1, n // seqs, dtype=torch.int32, device=DEV)
        slots = torch.arange(seqs, dtype=torch.int32, device=DEV)
        ms = timed(lambda: ops.mlstm_gates(z, bi, bfg, 15.0, state, cu, slots, heads, 128, 128))
        row(what, "matrix memory: gates, running maximum, keep / take / floor", ms, n * heads * (8 + 12))
        keep, take, floor = ops.mlstm_gates(z, bi, bfg, 15.0, state, cu, slots, heads, 128, 128)
        ms = timed(lambda: ops.mlstm_recurrence(proj, 0, hd, 2 * hd, 128 ** -0.5, keep, take, state, cu, slots, heads, 128, 128))
        flops = n * heads * 128 * 129 * 2 * 3
        row(what, "matrix memory: recurrence (S and n)", ms, n * (3 * hd * 2 + hd * 4 + heads * 12) + 2 * state.numel() * 4,
            f"{flops / ms / 1e9:,.1f} TFLOP/s float32 of the recurrence's own arithmetic")
        o, nq = ops.mlstm_recurrence(proj, 0, hd, 2 * hd, 128 ** -0.5, keep, take, state, cu, slots, heads, 128, 128)
        wn = rnd(hd)
        ms = timed(lambda: ops.mlstm_out_norm(o, nq, floor, proj, 3 * hd, wn, 1e-6, bf))
        row(what, "matrix memory: division, output norm and gate", ms, n * hd * (4 + 2 + 2))
        C, s_len = 3 * hd, heads * 128 * 128
        dstate = torch.zeros(seqs, s_len + 3 * C, device=DEV)
        dproj, taps = rnd(n, C + heads + 128), rnd(C, 4, dt=torch.float32)
        a_pre, dtb, alog = rnd(n, hd, dt=torch.float32), rnd(hd, dt=torch.float32), rnd(heads, dt=torch.float32)
        sotd = torch.repeat_interleave(torch.arange(seqs, device=DEV), n // seqs).to(torch.int32)
        ms = timed(lambda: ops.delta_prep(dproj, 0, C, taps, dstate, s_len, a_pre, dtb, alog, cu, sotd, slots, heads, heads, 128, 128))
        row(what, "like: delta rule: convolution, unit q/k, beta, decay", ms, n * (C * 2 + hd * 4 + (C + hd + heads) * 4))
        q, k, v, beta, decay = ops.delta_prep(dproj, 0, C, taps, dstate, s_len, a_pre, dtb, alog, cu, sotd, slots, heads, heads, 128, 128)
        ms = timed(lambda: ops.delta_recurrence(q, k, v, beta, decay, dstate, cu, slots, heads, heads, 128, 128, single_tokens=seqs == n))
        row(what, "like: delta rule: recurrence", ms, n * (C + hd + heads + hd) * 4 + 2 * seqs * s_len * 4,
            f"{n * heads * 128 * 128 * 2 * 3 / ms / 1e9:,.1f} TFLOP/s float32")
        og, gate, wn1 = rnd(n, hd, dt=torch.float32), rnd(n, hd), rnd(128)
        ms = timed(lambda: ops.delta_out_norm(og, gate, wn1, 1e-5, 128, bf))
        row(what, "like: delta rule: output norm and gate", ms, n * hd * (4 + 2 + 2))
        # routing and the experts
        xr, wr = rnd(n, width, dt=torch.float32), rnd(8, width)
        ms = timed(lambda: ops.router_plan(xr, wr, 2, ops.router_groups(4, 2), 1.5))
        row(what, "router: 8 experts in 4 groups, 2 kept, 2 chosen; plan", ms, n * width * 4 + 8 * width * 2)
        ms = timed(lambda: ops.router_plan(xr, wr, 2, 0, 1.0))
        row(what, "like: router without groups; plan", ms, n * width * 4 + 8 * width * 2)
        ids, scores, plan = ops.router_plan(xr, wr, 2, ops.router_groups(4, 2), 1.5)
        xe = rnd(n, width)
        e_ff = ff // 2
        w_up, w_gate, w_down = rnd(8, e_ff, width), rnd(8, e_ff, width), rnd(8, width, e_ff)
        ones = torch.ones_like(scores)
        if n * 2 > 10:
            def experts_relu2():
                return ops.moe_down_tc(ops.moe_up_relu2_tc(xe, plan, 2, w_up), w_down, plan)

            def experts_swiglu():
                return ops.moe_down_tc(ops.moe_gate_up_tc(xe, plan, 2, w_gate, w_up, scores), w_down, plan)
        else:
            def experts_relu2():
                return ops.moe_down(ops.moe_gate_up(xe, plan, 2, None, w_up, ones, True, "relu2"), w_down, plan, True)

            def experts_swiglu():
                return ops.moe_down(ops.moe_gate_up(xe, plan, 2, w_gate, w_up, scores, True), w_down, plan, True)
        touched = min(8, n * 2)
        ms = timed(experts_relu2)
        fl = n * 2 * 2 * 2 * width * e_ff
        row(what, "experts without a gate branch (up, squared relu, down)", ms, touched * 2 * e_ff * width * 2 + n * 2 * (width * 6 + e_ff * 4),
            f"{fl / ms / 1e9:,.0f} TFLOP/s bf16")
        ms = timed(experts_swiglu)
        row(what, "like: experts with gate and up (SwiGLU), down", ms, touched * 3 * e_ff * width * 2 + n * 2 * (width * 6 + e_ff * 4),
            f"{n * 2 * 3 * 2 * width * e_ff / ms / 1e9:,.0f} TFLOP/s bf16")
    ops.check_tc_status()
    # attention with the sink term beside the same kernels without it
    for n, what in ((tokens, "prefill"), (batch, "decode")):
        cached = 0 if what == "prefill" else context
        pages = (cached + n) // PAGE + 2
        kp, vp = (rnd(pages, nkv, PAGE, 128) for _ in range(2))
        q = rnd(n, heads, 128)
        if what == "prefill":
            pos = torch.arange(n, dtype=torch.int32, device=DEV)
            table = torch.arange(pages, dtype=torch.int32, device=DEV).view(1, pages)
            cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
            for sink in (True, False):
                ms = timed(lambda: ops.prefill_attention_tc(q, kp, vp, table, cu, pos, 1, n, 8192, 0, 128 ** -0.5, sink=sink))
                row(what, ("attention over the prompt's own keys, with the sink term" if sink else "like: the same kernel without it"), ms,
                    n * (heads * 2 + 2 * nkv) * 128 * 2, f"{4 * heads * 128 * n * n / 2 / ms / 1e9:,.0f} TFLOP/s bf16")
        else:
            pos = torch.full((n,), cached, dtype=torch.int32, device=DEV)
            table = torch.arange(pages, dtype=torch.int32, device=DEV).view(1, pages).repeat(n, 1).contiguous()
            seq = torch.arange(n, dtype=torch.int32, device=DEV)
            for sink in (True, False):
                ms = timed(lambda: ops.decode_attention(q, kp, vp, table, seq, pos, 8192, 0, 128 ** -0.5, cached + 1, sink=sink))
                row(what, ("attention of single tokens over the cache, with the sink term" if sink else "like: the same kernels without it"), ms,
                    2 * (cached + 1) * nkv * 128 * 2, "every request reads the same pages here: they come from L2")
    ops.check_tc_status()
    print("\n| step | kernel | us | MB that must move | GB/s | of the copy peak | |\n|---|---|---|---|---|---|---|")
    print("\n".join(rows))


def case_fidatar_step(tokens=2048, batch=8, context=4096, width=2048, heads=16, ff=8192, layers=4):
    """One Fidatar prompt step and three decode steps with every kernel launched on its own (no captured graph):
    for a launch list under ncu."""
    import torch

    from hi_b200.engine.core import Engine, StepEntry

    eng = Engine.from_config(_fidatar_config(width, heads, ff, layers), seed=0, dtype="bfloat16", device=DEV, kv_page_size=PAGE,
                             kv_cache_tokens=batch * (context + 256) + tokens + 256, max_active_requests=batch + 1,
                             use_cuda_graphs=False)
    g = torch.Generator().manual_seed(0)
    for rep in range(2):
        eng.step([StepEntry("p", torch.randint(0, eng.vocab_size, (tokens,), generator=g).tolist(), [tokens - 1])])
        eng.finish("p")
    for i in range(batch):
        eng.assume_cached(i, context)
    for _ in range(3):
        eng.step([StepEntry(i, [int(torch.randint(0, eng.vocab_size, (1,), generator=g))], [0]) for i in range(batch)])
    torch.cuda.synchronize()


def case_mlstm_recurrence(tokens=2048, heads=16, seqs=1, dim=128, vdim=128):
    """The matrix memory's recurrence alone, each of its register layouts twice: for ncu, and timed."""
    import torch

    from hi_b200.kernels import ops

    dg = torch.Generator(device=DEV).manual_seed(0)
    n = tokens * seqs
    proj = (torch.randn(n, heads * (2 * dim + vdim), device=DEV, generator=dg) * 0.5).to(torch.bfloat16)
    keep = torch.rand(n, heads, device=DEV) * 0.2 + 0.8
    take = torch.rand(n, heads, device=DEV)
    state = torch.zeros(seqs, ops.mlstm_state_floats(heads, dim, vdim), device=DEV)
    cu = torch.arange(0, n + 1, tokens, dtype=torch.int32, device=DEV)
    slots = torch.arange(seqs, dtype=torch.int32, device=DEV)
    for rows in (4, 8, 16, 32):
        if 32 * rows < dim:
            continue
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        args = (proj, 0, heads * dim, 2 * heads * dim, dim ** -0.5, keep, take, state, cu, slots, heads, dim, vdim, rows)
        ops.mlstm_recurrence(*args)
        a.record()
        ops.mlstm_recurrence(*args)
        b.record()
        torch.cuda.synchronize()
        print(f"{rows} rows a lane: {a.elapsed_time(b) * 1e3:.1f} us")


def _timeline(run, warm, what):
    """Kernel starts and ends of one step from the profiler's activity records (real durations, with
    what runs beside what), as markdown: the first two layers' launches, then totals by kernel."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    for _ in range(warm):
        run()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        run()
        torch.cuda.synchronize()
    evs = [e for e in prof.events() if e.device_type.name == "CUDA" and "emcpy" not in e.name and "emset" not in e.name]
    evs.sort(key=lambda e: e.time_range.start)
    name = lambda e: e.name.replace("void ", "").replace("(anonymous namespace)::", "").split("(")[0][:58]
    t0 = evs[0].time_range.start
    span = evs[-1].time_range.end - t0
    print(f"{what}: {len(evs)} kernels in {span:.0f} us\n")
    print("| start us | end us | us | kernel |\n|---|---|---|---|")
    norms = 0
    for e in evs:
        norms += "add_rmsnorm" in e.name
        if norms > 5:                       # two layers: four norms, then the third layer's first
            break
        print(f"| {e.time_range.start - t0:.1f} | {e.time_range.end - t0:.1f} | {e.time_range.end - e.time_range.start:.1f} | {name(e)} |")
    agg = {}
    for e in evs:
        a = agg.setdefault(name(e), [0, 0.0])
        a[0] += 1
        a[1] += e.time_range.end - e.time_range.start
    print("\n| kernel | launches | us in all | us each |\n|---|---|---|---|")
    for k, (c, v) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        print(f"| {k} | {c} | {v:.1f} | {v / c:.1f} |")


def case_decode_timeline(batch=8, context=8192, layers=4):
    """One captured decode step of ``batch`` requests at ``context`` cached tokens: when each kernel ran."""
    import torch

    from hi_b200.engine.core import StepEntry

    eng = _case_engine(layers, batch * (context + 128), batch + 1)
    eng.use_cuda_graphs = True
    for view in eng.cache.views.values():
        view.k_pages.normal_(); view.v_pages.normal_()
    for i in range(batch):
        eng.assume_cached(i, context - 16)
    g = torch.Generator().manual_seed(0)
    step = lambda: eng.step([StepEntry(i, [int(torch.randint(0, 202048, (1,), generator=g))], [0]) for i in range(batch)])
    _timeline(step, 6, f"decode step, {batch} requests x {context} cached tokens, {layers} Scout-sized layers, captured graph")


def case_prefill_timeline(tokens=2048, layers=4):
    """One prompt of ``tokens`` tokens in one step: when each kernel ran."""
    import torch

    from hi_b200.engine.core import StepEntry

    eng = _case_engine(layers, tokens + 128, 2)
    g = torch.Generator().manual_seed(0)
    count = [0]

    def step():
        count[0] += 1
        eng.step([StepEntry(count[0], torch.randint(0, 202048, (tokens,), generator=g).tolist(), [tokens - 1])])
        eng.finish(count[0])

    _timeline(step, 3, f"prefill step, one prompt of {tokens} tokens, {layers} Scout-sized layers")


CASES = {"sweep": case_sweep, "decode_timeline": case_decode_timeline, "prefill_timeline": case_prefill_timeline, "decode_attention": case_decode_attention, "decode_attention_fused": case_decode_attention_fused, "expert_gemv": case_expert_gemv, "expert_tc": case_expert_tc,
         "prefill_attention": case_prefill_attention, "decode_step": case_decode_step, "prefill_step": case_prefill_step,
         "vinurax": case_vinurax, "delta_recurrence": case_delta_recurrence,
         "vinurax_step": case_vinurax_step, "fidatar": case_fidatar, "fidatar_step": case_fidatar_step,
         "mlstm_recurrence": case_mlstm_recurrence, "surinex": case_surinex, "surinex_step": case_surinex_step,
         "bezasun": case_bezasun, "bezasun_step": case_bezasun_step, "bezasun_attention": case_bezasun_attention}


if __name__ == "__main__":
    sys.exit(main())
