"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl reference]
                    [--shape 8b|14b|32b] [--prompt-len P] [--new-tokens T] [--workload decode|mixed]
                    [--design fumanex|kamelorn|muzopel|deletar]

The model has the layer sizes of Qwen3-8B with seeded random weights made on the device; prompts
are seeded random token ids.  A step is one decode step of ``--batch`` requests whose prompts
(2,048 tokens each) were prefilled before the timed region.  ``value`` is decoded tokens per second
timed on the device around K steps of the step function plus the sampling kernel; ``e2e`` is the
same through ``LLMEngine.step()`` with host token ids in and sampled tokens out every step.
Every decode step reads all weights (15 GB, far larger than the 126 MB L2), so nothing is served
from L2 between iterations.  12vivi/tandem measures the same quantities with
benchmarks/bench_offline.py:54-62 (random ids, greedy, ignore_eos).

``--shape`` takes the layer sizes of Qwen3-14B or Qwen3-32B instead (the default line is the one
of Qwen3-8B).  ``--workload mixed`` runs requests with prompts of random lengths (128 to 4,096
tokens) through the scheduler with 128 greedy tokens each, prompt portions of up to 2,048 tokens
beside decoded tokens, and prints its own line: generated and processed tokens per second of
wall-clock time (benchmarks/bench_offline.py:64-86 of 12vivi/tandem).

``--design fumanex`` prints a line of its own: prefill and decode throughput of Fumanex models with
random weights at two sizes beside Qwen3 models of equal width, heads, layers and feed-forward
weights, and the design's own kernels against their rooflines.  ``--design kamelorn`` does the same for Kamelorn
models (state-space layers, attention over a cached latent, dense and routed feed-forwards, a residual of two
streams), ``--design muzopel`` for Muzopel models (norms behind the sublayers, short convolutions, a weighted sum over
the layers' results, latent attention, experts of two matrices) beside Kamelorn models with latent attention and experts
of equal size in every layer, ``--design deletar`` for Deletar models (windowed attention whose queries and keys are
convolved, normed and rotated, norms on both sides of the sublayers, experts named by a table of token ids) beside Fumanex
models with windowed attention in every layer and as many parameters.  The default line is untouched.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen3-8B layer sizes (the configuration the benchmark is quoted on)
QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936,
                rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096)
QWEN3_14B = dict(QWEN3_8B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600)
SHAPES = {"8b": ("Qwen3-8B shape", QWEN3_8B), "14b": ("Qwen3-14B shape", QWEN3_14B), "32b": ("Qwen3-32B shape", QWEN3_32B)}
PROMPT, NEW_TOKENS, PAGE = 2048, 256, 16


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d.get("hbm_gbs", 6650.0)), tflops=float(d.get("bf16_tflops", 1590.0)),
                    tflops_sustained=float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", 1590.0))), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while the timed regions run."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.proc.wait()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7 or not f[0].isdigit():
                continue
            sm.append(int(f[0])), mx.append(int(f[1]))
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.remove(self.path)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_engine(shape: dict, layers: int, max_seqs: int, tokens_per_seq: int, cuda_graph: bool = True,
                 policy: str = "prefill_first", pages: int = 0):
    from tandem_b200 import EngineConfig, LLMEngine
    from tandem_b200.engine.core import random_model

    max_len = max(4096, -(-tokens_per_seq // PAGE) * PAGE)
    decoder, cfg = random_model(dict(shape, max_position_embeddings=max_len), seed=0, dtype="bfloat16", num_layers=layers)
    pages = pages or max_seqs * (-(-tokens_per_seq // PAGE)) + 8
    eng = LLMEngine(EngineConfig(model="", dtype="bfloat16", block_size=PAGE, num_kv_blocks=pages, max_num_seqs=max_seqs,
                                 max_num_batched_tokens=2048, max_model_len=max_len, schedule_policy=policy,
                                 cuda_graph=cuda_graph, cuda_graph_max_bs=max_seqs),
                    decoder=decoder, model_config=cfg, load_tokenizer=False)
    return eng


def prompts(batch: int, seed: int = 0, length: int = PROMPT) -> list:
    import torch

    g = torch.Generator().manual_seed(seed)
    return [torch.randint(10, 100000, (length,), generator=g).tolist() for _ in range(batch)]


def decode_bytes(eng, batch: int, context: int) -> float:
    """What one decode step has to read: every weight it uses once (the embedding table is only
    gathered from) and the cache of the live requests."""
    from tandem_b200.engine.core import kv_bytes_per_token

    d = eng.decoder
    weights = d.parameter_bytes - d.embedding.numel() * d.embedding.element_size() * (0 if d.head is d.embedding else 1)
    return weights + batch * context * kv_bytes_per_token(d)


def measure_decode(eng, batch: int, steps: int, warmup: int, prompt_len: int = PROMPT, new_tokens: int = NEW_TOKENS) -> dict:
    """Device time of ``steps`` decode steps of ``batch`` requests just behind their prompts of
    ``prompt_len`` tokens, then the same through LLMEngine.step()."""
    import torch

    from tandem_b200 import SamplingParams
    from tandem_b200.kernels import ops

    sp = SamplingParams(max_tokens=new_tokens + steps + 2 * warmup + 16, temperature=0.0, ignore_eos=True)
    for p in prompts(batch, seed=batch, length=prompt_len):
        eng.add_request(p, sp)
    while any(not r.is_decoding for r in eng.requests.values()) or eng.scheduler.waiting:
        eng.step()  # prefill, untimed
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()

    # end to end: host ids in, sampled tokens out, every step
    t0 = time.perf_counter()
    for _ in range(steps):
        eng.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    h2d = eng.executor.h2d_bytes_last  # what one of these steps copied to the device: its batch description
    eng.drain()  # the step in flight (overlap scheduling)

    # device-timed: the step function and the sampling kernel back to back, no host read in between
    plan = eng.scheduler.schedule()
    entries = eng.entries_of(plan)
    for e in entries:
        e.want = [0]
    runner = eng.graphs if (eng.graphs is not None and eng.graphs.takes(entries)) else eng.executor
    context = max(r.num_computed_tokens for r in eng.requests.values())
    for _ in range(max(1, warmup)):
        ops.argmax(runner.run(entries))
    torch.cuda.synchronize()
    before = ops.launches
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        ops.argmax(runner.run(entries))
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    launches = (ops.launches - before) // steps if eng.graphs is None else eng.graphs.launches_per_replay(entries) + 1
    for rid in list(eng.requests):
        eng.abort_request(rid)
    assert eng.cache.all_free()
    return dict(ms=ms, tok_s=batch * 1000.0 / ms, e2e_tok_s=batch * steps / e2e_s, e2e_ms=e2e_s * 1000 / steps,
                context=context, launches=launches, bytes=decode_bytes(eng, batch, context), h2d=h2d)


def measure_prefill(eng, warmup: int, reps: int = 3) -> dict:
    import torch

    from tandem_b200.engine.executor import StepEntry

    toks = prompts(1, seed=99)[0]
    times = []
    for i in range(warmup + reps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        eng.executor.step([StepEntry(f"p{i}", toks, [PROMPT - 1])], end=[f"p{i}"])
        stop.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(start.elapsed_time(stop))
    ms = sorted(times)[len(times) // 2]
    c = eng.model_config
    per_layer = c.hidden_size * (c.q_size + 2 * c.kv_size) + c.q_size * c.hidden_size + 3 * c.hidden_size * c.intermediate_size
    linear = 2.0 * PROMPT * c.num_hidden_layers * per_layer + 2.0 * c.hidden_size * c.vocab_size  # one row of logits
    attn = c.num_hidden_layers * 4.0 * c.num_attention_heads * c.head_dim * PROMPT * (PROMPT + 1) / 2
    return dict(ms=ms, tok_s=PROMPT * 1000.0 / ms, flops=linear + attn)


def measure_mixed(eng, num_requests: int, new_tokens: int, seed: int = 0) -> dict:
    """Requests with prompts of random lengths through the scheduler: portions of prompts beside
    decoded tokens, until every request has its ``new_tokens``.  Wall-clock time."""
    import torch

    from tandem_b200 import SamplingParams
    from tandem_b200.kernels import ops

    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(128, 4097, (num_requests,), generator=g).tolist()
    sp = SamplingParams(max_tokens=new_tokens, temperature=0.0, ignore_eos=True)
    result = {}
    for rep in range(2):  # the first pass builds graphs and measures product dispatch; the second is timed
        for n in lengths:
            eng.add_request(torch.randint(10, 100000, (n,), generator=g).tolist(), sp)
        torch.cuda.synchronize()
        before, steps, t0 = ops.launches, 0, time.perf_counter()
        while eng.has_unfinished_requests():
            eng.step()
            steps += 1
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        assert eng.cache.all_free()
        result = dict(seconds=seconds, steps=steps, launches=ops.launches - before, prompt_tokens=sum(lengths),
                      new_tokens=num_requests * new_tokens, preemptions=eng.scheduler.num_preemptions)
    return result


def measure_extras(steps: int, warmup: int) -> dict:
    """The two other workloads the benchmark is quoted on, each with a model of its own, as flat
    keys beside the headline: decode at batch 8 at Qwen3-32B sizes (1,024-token prompts), and 32
    requests with prompts of 128 to 4,096 tokens and 128 new tokens each at Qwen3-14B sizes."""
    import gc

    import torch

    out: dict = {}
    pk = peaks()

    def release():
        gc.collect()
        torch.cuda.empty_cache()

    try:
        t0 = time.perf_counter()
        eng = build_engine(QWEN3_32B, QWEN3_32B["num_hidden_layers"], 8, 1024 + 128 + steps + 2 * warmup + 32)
        r = measure_decode(eng, 8, steps, warmup, 1024, 128)
        out.update({"qwen3_32b_layers": eng.model_config.num_hidden_layers, "qwen3_32b_decode_b8_tok_s": round(r["tok_s"], 1),
                    "qwen3_32b_decode_b8_ms": round(r["ms"], 4), "qwen3_32b_decode_b8_e2e_tok_s": round(r["e2e_tok_s"], 1),
                    "qwen3_32b_decode_b8_hbm_frac": round(r["bytes"] / (r["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
                    "qwen3_32b_seconds": round(time.perf_counter() - t0, 1)})
        del eng
    except Exception as exc:  # the headline stands without it
        out["qwen3_32b_error"] = f"{type(exc).__name__}: {exc}"[:200]
    release()
    try:
        t0 = time.perf_counter()
        eng = build_engine(QWEN3_14B, QWEN3_14B["num_hidden_layers"], 32, 4096 + 128)
        r = measure_mixed(eng, 32, 128)
        out.update({"qwen3_14b_layers": eng.model_config.num_hidden_layers,
                    "qwen3_14b_mixed_generated_tok_s": round(r["new_tokens"] / r["seconds"], 1),
                    "qwen3_14b_mixed_processed_tok_s": round((r["new_tokens"] + r["prompt_tokens"]) / r["seconds"], 1),
                    "qwen3_14b_mixed_seconds": round(r["seconds"], 3), "qwen3_14b_mixed_steps": r["steps"],
                    "qwen3_14b_mixed_preemptions": r["preemptions"], "qwen3_14b_seconds": round(time.perf_counter() - t0, 1)})
        del eng
    except Exception as exc:
        out["qwen3_14b_error"] = f"{type(exc).__name__}: {exc}"[:200]
    release()
    return out


def main_mixed(args, name: str, shape: dict) -> int:
    pk = peaks()
    per_request = 4096 + args.new_tokens
    eng = build_engine(shape, args.layers, args.batch, per_request, not args.no_cuda_graph, policy=args.policy)
    sampler = ClockSampler()
    sampler.start()
    r = measure_mixed(eng, args.batch, args.new_tokens)
    clocks = sampler.stop()
    c = eng.model_config
    out = {
        "metric": f"generated tok/s, {args.batch} requests with prompts of 128-4,096 tokens, {name} (one B200)",
        "value": round(r["new_tokens"] / r["seconds"], 1), "unit": "tok/s", "n_gpus": 1, "steps": r["steps"],
        "processed_tok_s": round((r["new_tokens"] + r["prompt_tokens"]) / r["seconds"], 1), "seconds": round(r["seconds"], 3),
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic: seeded random weights N(0,0.02) and random token ids",
        "config": {"model": name, "layers": c.num_hidden_layers, "layers_full": shape["num_hidden_layers"],
                   "hidden": c.hidden_size, "q_heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
                   "head_dim": c.head_dim, "intermediate": c.intermediate_size, "vocab": c.vocab_size,
                   "requests": args.batch, "prompt_tokens": r["prompt_tokens"], "new_tokens": r["new_tokens"],
                   "token_budget": 2048, "policy": args.policy, "page_size": PAGE, "preemptions": r["preemptions"],
                   "peaks": pk["source"]},
        "gpu_launches": r["launches"], "clocks": clocks,
    }
    print(json.dumps(out))
    return 0


# ---------------------------------------------------------------------------------------------
# --design fumanex: the hybrid design beside Qwen3 at equal size
def fumanex_shape(width: int, heads: int, kv_heads: int, ff: int, layers: int, window: int = 1024) -> dict:
    """Layers of attention (window, kept first tokens, sink, bias by distance, mixed values), lightning and
    retention in turn, head size 128 throughout; the dense feed-forward of two matrices has the weights of
    the gated one of three that the Qwen3 model beside it has."""
    att = dict(type="attention", mixer=dict(heads=heads, kv_heads=kv_heads, dim=128, vdim=128, scale=128 ** -0.5, softcap=30.0,
                                            bias_max=window, v_mix=True, mask=dict(size=window, keep_first=4)), mlp=dict(kind="dense", ff=ff))
    lig = dict(type="lightning", mixer=dict(heads=heads, dim=128, vdim=128, decay=[1.0 - 2.0 ** -(5 + 3 * i / heads) for i in range(heads)]),
               mlp=dict(kind="dense", ff=ff))
    ret = dict(type="retention", mixer=dict(heads=heads, dim=128, vdim=128, decay=[1.0 - 2.0 ** -(5 + 3 * i / heads) for i in range(heads)],
                                            rot=dict(dims=64, base=1e6)), mlp=dict(kind="dense", ff=ff))
    return dict(architecture="Fumanex", vocab=151936, width=width, embedding=dict(scale=1.0), logit_scale=1.0, norm=dict(eps=1e-6),
                layers=[(att, lig, att, ret)[i % 4] for i in range(layers)])


DESIGN_SIZES = {
    "2k": (fumanex_shape(2048, 16, 4, 8256, 8), dict(QWEN3_8B, num_hidden_layers=8, hidden_size=2048, num_attention_heads=16,
                                                    num_key_value_heads=4, intermediate_size=5504)),
    "4k": (fumanex_shape(4096, 32, 8, 18432, 8), dict(QWEN3_8B, num_hidden_layers=8)),
}


def kamelorn_shape(width: int, heads: int, ff: int, layers: int, experts: int, top: int, expert_ff: int, groups: int) -> dict:
    """Three state-space layers to one layer of attention over a latent; dense and routed feed-forwards in turn; a residual
    of two streams.  State-space: inner width twice the model's in heads of 64, 128 state rows, four taps.  Latent: 96
    numbers + 32 rotated, heads of 64 + 32 query dims and 64 value dims (the sizes the tensor-core tile kernel takes)."""
    def mamba(mlp):
        return dict(type="mamba2", mixer=dict(heads=2 * width // 64, vdim=64, state=128, groups=groups, conv=4, norm_groups=1), mlp=mlp)

    def latent(mlp):
        return dict(type="latent_attention", mixer=dict(heads=heads, dim=64, rot_dim=32, vdim=64, kv_rank=96, scale=96 ** -0.5,
                                                        rot=dict(dims=32, base=1e6)), mlp=mlp)

    dense = dict(kind="dense", ff=ff)
    routed = dict(kind="moe", expert=dict(ff=expert_ff), router=dict(experts=experts, top=top, scale=1.0))
    four = [mamba(dense), mamba(routed), latent(dense), mamba(routed)]
    return dict(architecture="Kamelorn", vocab=151936, width=width, embedding=dict(scale=1.0), norm=dict(eps=1e-6), residual_mult=1.0,
                streams=2, layers=[four[i % 4] for i in range(layers)])


KAMELORN_SIZES = {
    "2k": (kamelorn_shape(2048, 16, 5504, 8, 16, 2, 1408, 1), dict(QWEN3_8B, num_hidden_layers=8, hidden_size=2048, num_attention_heads=16,
                                                                  num_key_value_heads=4, intermediate_size=5504)),
    "4k": (kamelorn_shape(4096, 32, 12288, 8, 32, 4, 2048, 8), dict(QWEN3_8B, num_hidden_layers=8)),
}


def main_kamelorn(args) -> int:
    import gc

    import torch

    from tandem_b200.kernels import microbench

    pk = peaks()
    sampler = ClockSampler()
    sampler.start()
    sizes = {}
    launches = 0
    for size, (kam, qwen) in KAMELORN_SIZES.items():
        row = {}
        for name, config in (("kamelorn", kam), ("qwen3", qwen)):
            eng = design_engine(config, args.batch, PROMPT + NEW_TOKENS + args.steps + 2 * args.warmup + 32)
            d = measure_decode(eng, args.batch, args.steps, args.warmup, PROMPT, NEW_TOKENS)
            ms = design_prefill_ms(eng, args.warmup)
            row[name] = {"prefill_tok_s": round(PROMPT * 1000.0 / ms, 1), "prefill_ms": round(ms, 3), "decode_tok_s": round(d["tok_s"], 1),
                         "decode_ms_per_step": round(d["ms"], 4), "decode_e2e_tok_s": round(d["e2e_tok_s"], 1),
                         "launches_per_decode_step": int(d["launches"]), "parameters": eng.decoder.num_parameters}
            launches += int(d["launches"]) * args.steps
            del eng, d
            gc.collect()
            torch.cuda.empty_cache()
        sizes[size] = row
    with torch.inference_mode():
        sel = microbench.selective_case(PROMPT, args.batch, 128, 8, 128, 64, 20, True)
        rec = microbench.recurrence_case(PROMPT, args.batch, 32, 128, 128, 20, True)
        att = microbench.sink_attention_case(PROMPT, args.batch, PROMPT, 32, 1, 128, 96, PAGE, None, 0, 20, True)
        exp = microbench.experts_case(PROMPT, args.batch, 4096, 2048, 32, 4, 20, True)
    kernels = {
        "selective_scan_prompt_2048": {"us": round(sel["prefill_us"], 1), "tflops_fp32": round(sel["prefill_tflops"], 2)},
        "selective_scan_decode_b%d" % args.batch: {"us": round(sel["decode_us"], 1), "gbs": round(sel["decode_gbs"], 1),
                                                   "frac_of_hbm": round(sel["decode_gbs"] / pk["hbm_gbs"], 4)},
        "decay_recurrence_prompt_2048": {"us": round(rec["prefill_us"], 1), "tflops_fp32": round(rec["prefill_tflops"], 2)},
        "decay_recurrence_decode_b%d" % args.batch: {"us": round(rec["decode_us"], 1), "gbs": round(rec["decode_gbs"], 1),
                                                     "frac_of_hbm": round(rec["decode_gbs"] / pk["hbm_gbs"], 4)},
        "latent_attention_tiles_prompt_2048": {"us": round(att["prefill_us"], 1), "tflops": round(att["prefill_tflops"], 1),
                                               "frac_of_bf16_peak": round(att["prefill_tflops"] / pk["tflops"], 4)},
        "latent_attention_decode_b%d" % args.batch: {"us": round(att["decode_us"], 1), "gbs": round(att["decode_gbs"], 1),
                                                     "frac_of_hbm": round(att["decode_gbs"] / pk["hbm_gbs"], 4)},
        "experts_tiles_2048_tokens": {"us": round(exp["prefill_us"], 1), "tflops": round(exp["prefill_tflops"], 1),
                                      "frac_of_bf16_peak": round(exp["prefill_tflops"] / pk["tflops"], 4)},
        "experts_decode_b%d" % args.batch: {"us": round(exp["decode_us"], 1), "gbs": round(exp["decode_gbs"], 1),
                                            "frac_of_hbm": round(exp["decode_gbs"] / pk["hbm_gbs"], 4)},
    }
    clocks = sampler.stop()
    k4 = sizes["4k"]["kamelorn"]
    print(json.dumps({
        "metric": f"decode tok/s at batch {args.batch}, Kamelorn (8 layers, width 4096), {PROMPT:,}-token prompts (one B200)",
        "value": k4["decode_tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": k4["decode_ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights and random token ids",
        "config": {"model": "Kamelorn beside Qwen3 at equal width and depth", "global_batch": args.batch, "seq_len": PROMPT, "page_size": PAGE,
                   "parallelism": "single GPU", "l2": "inputs larger than L2: each step streams every weight", "peaks": pk["source"]},
        "e2e": {"value": k4["decode_e2e_tok_s"], "unit": "tok/s"}, "gpu_launches": launches,
        "sizes": sizes, "kernels": kernels, "clocks": clocks}))
    return 0


def muzopel_shape(width: int, heads: int, layers: int, experts: int, top: int, expert_ff: int, identity: int, q_rank: int) -> dict:
    """Latent attention with query latents, stretched frequencies and a gate per head, then two layers with plain queries,
    in turn; every layer with routed experts of two matrices (``identity`` router outputs more stand for experts that return
    their input), convolutions of four taps, norms in four groups.  Latent: 96 numbers + 32 rotated, heads of 64 + 32 query
    dims and 64 value dims (the sizes the tensor-core tile kernel takes)."""
    rot = dict(dims=32, base=1e6)
    mlp = dict(kind="moe", expert=dict(ff=expert_ff), router=dict(experts=experts, identity=identity, top=top))
    sizes = dict(heads=heads, dim=64, rot_dim=32, vdim=64, kv_rank=96, scale=96 ** -0.5)
    first = dict(type="latent_attention", mlp=mlp,
                 mixer=dict(sizes, q_rank=q_rank, rot=dict(rot, scaling=dict(factor=8.0, original=4096, fast=32.0, slow=1.0))))
    second = dict(type="latent_attention_2", mixer=dict(sizes, rot=rot), mlp=mlp)
    return dict(architecture="Muzopel", vocab=151936, width=width, norm=dict(eps=1e-6, groups=4), canon=dict(taps=4), logit_softcap=30.0,
                layers=[(first, second, second)[i % 3] for i in range(layers)])


def kamelorn_latent_shape(width: int, heads: int, layers: int, experts: int, top: int, expert_ff: int) -> dict:
    """The closest model the package had: Kamelorn with latent attention of the same sizes in every layer and gated routed
    experts (three matrices of two thirds the width of Muzopel's two), one residual stream."""
    layer = dict(type="latent_attention", mixer=dict(heads=heads, dim=64, rot_dim=32, vdim=64, kv_rank=96, scale=96 ** -0.5,
                                                    rot=dict(dims=32, base=1e6)),
                 mlp=dict(kind="moe", expert=dict(ff=expert_ff), router=dict(experts=experts, top=top, scale=1.0)))
    return dict(architecture="Kamelorn", vocab=151936, width=width, embedding=dict(scale=1.0), norm=dict(eps=1e-6), residual_mult=1.0,
                layers=[layer] * layers)


MUZOPEL_SIZES = {
    "2k": (muzopel_shape(2048, 16, 8, 16, 2, 2112, 2, 512), kamelorn_latent_shape(2048, 16, 8, 16, 2, 1408)),
    "4k": (muzopel_shape(4096, 32, 8, 32, 4, 3072, 2, 1024), kamelorn_latent_shape(4096, 32, 8, 32, 4, 2048)),
}


def main_muzopel(args) -> int:
    import gc

    import torch

    from tandem_b200.kernels import microbench

    pk = peaks()
    sampler = ClockSampler()
    sampler.start()
    sizes = {}
    launches = 0
    for size, (muz, kam) in MUZOPEL_SIZES.items():
        row = {}
        for name, config in (("muzopel", muz), ("kamelorn", kam)):
            eng = design_engine(config, args.batch, PROMPT + NEW_TOKENS + args.steps + 2 * args.warmup + 32)
            d = measure_decode(eng, args.batch, args.steps, args.warmup, PROMPT, NEW_TOKENS)
            ms = design_prefill_ms(eng, args.warmup)
            row[name] = {"prefill_tok_s": round(PROMPT * 1000.0 / ms, 1), "prefill_ms": round(ms, 3), "decode_tok_s": round(d["tok_s"], 1),
                         "decode_ms_per_step": round(d["ms"], 4), "decode_e2e_tok_s": round(d["e2e_tok_s"], 1),
                         "launches_per_decode_step": int(d["launches"]), "parameters": eng.decoder.num_parameters}
            launches += int(d["launches"]) * args.steps
            del eng, d
            gc.collect()
            torch.cuda.empty_cache()
        sizes[size] = row
    with torch.inference_mode():
        att = microbench.sink_attention_case(PROMPT, args.batch, PROMPT, 32, 1, 128, 96, PAGE, None, 0, 20, True)
        plain = microbench.experts_case(PROMPT, args.batch, 4096, 3072, 32, 4, 20, True, gated=False, identity=2)
        gated = microbench.experts_case(PROMPT, args.batch, 4096, 2048, 32, 4, 20, True)
        pn = microbench.post_norm_case(PROMPT, args.batch, 4096, 4, 4, 8, 20, True)

    def flops(r, which):
        return {"us": round(r[which + "_us"], 1), "tflops": round(r[which + "_tflops"], 1),
                "frac_of_bf16_peak": round(r[which + "_tflops"] / pk["tflops"], 4)}

    def stream(us, gbs):
        return {"us": round(us, 1), "gbs": round(gbs, 1), "frac_of_hbm": round(gbs / pk["hbm_gbs"], 4)}

    b = "decode_b%d" % args.batch
    kernels = {
        "latent_attention_tiles_prompt_2048": flops(att, "prefill"),
        "latent_attention_" + b: stream(att["decode_us"], att["decode_gbs"]),
        "experts_2_matrices_2048_tokens": flops(plain, "prefill"),
        "experts_3_matrices_2048_tokens": flops(gated, "prefill"),
        "experts_2_matrices_" + b: stream(plain["decode_us"], plain["decode_gbs"]),
        "experts_3_matrices_" + b: stream(gated["decode_us"], gated["decode_gbs"]),
    }
    for which, label in (("prefill", "prompt_2048"), ("decode", b)):
        for k in ("link_conv", "link_average", "conv", "add_rmsnorm"):
            kernels[f"{k}_{label}"] = stream(pn[f"{which}_{k}_us"], pn[f"{which}_{k}_gbs"])
        kernels[f"conv_state_{label}"] = {"us": round(pn[f"{which}_conv_state_us"], 1)}
    clocks = sampler.stop()
    m4 = sizes["4k"]["muzopel"]
    print(json.dumps({
        "metric": f"decode tok/s at batch {args.batch}, Muzopel (8 layers, width 4096), {PROMPT:,}-token prompts (one B200)",
        "value": m4["decode_tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": m4["decode_ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights and random token ids",
        "config": {"model": "Muzopel beside Kamelorn with latent attention and experts of equal size in every layer", "global_batch": args.batch,
                   "seq_len": PROMPT, "page_size": PAGE, "parallelism": "single GPU",
                   "l2": "inputs larger than L2: each step streams every weight", "peaks": pk["source"]},
        "e2e": {"value": m4["decode_e2e_tok_s"], "unit": "tok/s"}, "gpu_launches": launches,
        "sizes": sizes, "kernels": kernels, "clocks": clocks}))
    return 0


# --design deletar: windowed attention with prepared queries and keys, norms on both sides of the sublayers, experts named by a
# table of token ids, beside the package's other windowed-attention model at equal size
def deletar_shape(width: int, heads: int, kv_heads: int, ff: int, layers: int, experts: int, top: int, expert_ff: int, window: int = 1024) -> dict:
    """Four kinds of layer in turn, head size 128 throughout: keys for values with a norm over all heads (dense feed-forward);
    a norm per head, slowed frequencies and a sink (experts); a convolution of four taps on q, k and v (experts); a layer that
    borrows the second one's keys and values (dense).  Experts of two matrices plus a shared one of the same width."""
    sizes = dict(heads=heads, kv_heads=kv_heads, dim=128, vdim=128, scale=128 ** -0.5, mask=dict(size=window))
    rot = dict(dims=64, base=1e6)
    slowed = dict(rot, scaling=dict(factor=8.0, low=1.0, high=4.0, original=4096))
    dense = dict(kind="dense", ff=ff)
    routed = dict(kind="moe", expert=dict(ff=expert_ff), router=dict(experts=experts, top=top), shared=dict(ff=expert_ff))

    def four(i):
        return [dict(type="attention_2", mixer=dict(sizes, softcap=30.0, rot=rot), mlp=dense),
                dict(type="attention_3", mixer=dict(sizes, softcap=30.0, rot=slowed), mlp=routed),
                dict(type="attention", mixer=dict(sizes, conv=4, rot=rot), mlp=routed),
                dict(type="attention_3", mixer=dict(sizes, softcap=30.0, rot=slowed, kv_from=i + 1), mlp=dense)]

    return dict(architecture="Deletar", vocab=151936, width=width, embedding=dict(scale=1.0), norm=dict(eps=1e-6), logit_softcap=30.0,
                layers=[four(i - i % 4)[i % 4] for i in range(layers)])


def fumanex_attention_shape(width: int, heads: int, kv_heads: int, ff: int, layers: int, window: int = 1024) -> dict:
    """The closest model the package had: Fumanex with its windowed attention (sink, cap, bias by distance, unit-norm q and k)
    in every layer and a dense feed-forward of two matrices."""
    att = dict(type="attention", mixer=dict(heads=heads, kv_heads=kv_heads, dim=128, vdim=128, scale=128 ** -0.5, softcap=30.0,
                                            bias_max=window, v_mix=False, mask=dict(size=window, keep_first=4)), mlp=dict(kind="dense", ff=ff))
    return dict(architecture="Fumanex", vocab=151936, width=width, embedding=dict(scale=1.0), logit_scale=1.0, norm=dict(eps=1e-6),
                layers=[att] * layers)


# the dense width of the model beside it is chosen so that both have the same number of parameters (to within a percent)
DELETAR_SIZES = {
    "2k": (deletar_shape(2048, 16, 4, 8256, 8, 16, 2, 2112), fumanex_attention_shape(2048, 16, 4, 22208, 8)),
    "4k": (deletar_shape(4096, 32, 8, 18432, 8, 32, 4, 3072), fumanex_attention_shape(4096, 32, 8, 59904, 8)),
}


def main_deletar(args) -> int:
    import gc

    import torch

    from tandem_b200.kernels import microbench

    pk = peaks()
    sampler = ClockSampler()
    sampler.start()
    sizes = {}
    launches = 0
    for size, (dele, fum) in DELETAR_SIZES.items():
        row = {}
        for name, config in (("deletar", dele), ("fumanex", fum)):
            eng = design_engine(config, args.batch, PROMPT + NEW_TOKENS + args.steps + 2 * args.warmup + 32)
            d = measure_decode(eng, args.batch, args.steps, args.warmup, PROMPT, NEW_TOKENS)
            ms = design_prefill_ms(eng, args.warmup)
            row[name] = {"prefill_tok_s": round(PROMPT * 1000.0 / ms, 1), "prefill_ms": round(ms, 3), "decode_tok_s": round(d["tok_s"], 1),
                         "decode_ms_per_step": round(d["ms"], 4), "decode_e2e_tok_s": round(d["e2e_tok_s"], 1),
                         "launches_per_decode_step": int(d["launches"]), "parameters": eng.decoder.num_parameters}
            launches += int(d["launches"]) * args.steps
            del eng, d
            gc.collect()
            torch.cuda.empty_cache()
        sizes[size] = row
    with torch.inference_mode():
        wa = microbench.window_attention_case(PROMPT, args.batch, PROMPT, 4096, 32, 8, 128, 128, PAGE, 1024, 4, 20, True)
        fa = microbench.sink_attention_case(PROMPT, args.batch, PROMPT, 32, 8, 128, 128, PAGE, 1024, 4, 20, True)
        relu2 = microbench.experts_case(PROMPT, args.batch, 4096, 3072, 32, 4, 20, True, gated=False, activation="relu2")
        gelu = microbench.experts_case(PROMPT, args.batch, 4096, 3072, 32, 4, 20, True, gated=False)

    def flops(us, tflops):
        return {"us": round(us, 1), "tflops": round(tflops, 1), "frac_of_bf16_peak": round(tflops / pk["tflops"], 4)}

    def stream(us, gbs):
        return {"us": round(us, 1), "gbs": round(gbs, 1), "frac_of_hbm": round(gbs / pk["hbm_gbs"], 4)}

    b = "decode_b%d" % args.batch
    kernels = {
        "window_attention_tiles_prompt_2048": flops(wa["prefill_attention_us"], wa["prefill_attention_tflops"]),
        "fumanex_attention_tiles_prompt_2048": flops(fa["prefill_us"], fa["prefill_tflops"]),
        "window_attention_" + b: stream(wa["decode_attention_us"], wa["decode_attention_gbs"]),
        "fumanex_attention_" + b: stream(fa["decode_us"], fa["decode_gbs"]),
        "experts_relu2_2048_tokens": flops(relu2["prefill_us"], relu2["prefill_tflops"]),
        "experts_gelu_2048_tokens": flops(gelu["prefill_us"], gelu["prefill_tflops"]),
        "experts_relu2_" + b: stream(relu2["decode_us"], relu2["decode_gbs"]),
        "experts_gelu_" + b: stream(gelu["decode_us"], gelu["decode_gbs"]),
    }
    for which, label in (("prefill", "prompt_2048"), ("decode", b)):
        for k in ("prepare_whole", "prepare_head", "prepare_conv", "prep_unit", "norm_add_norm", "add_rmsnorm"):
            kernels[f"{k}_{label}"] = stream(wa[f"{which}_{k}_us"], wa[f"{which}_{k}_gbs"])
    clocks = sampler.stop()
    m4 = sizes["4k"]["deletar"]
    print(json.dumps({
        "metric": f"decode tok/s at batch {args.batch}, Deletar (8 layers, width 4096), {PROMPT:,}-token prompts (one B200)",
        "value": m4["decode_tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": m4["decode_ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights and random token ids",
        "config": {"model": "Deletar beside Fumanex with windowed attention in every layer, at equal size", "global_batch": args.batch,
                   "seq_len": PROMPT, "page_size": PAGE, "parallelism": "single GPU",
                   "l2": "inputs larger than L2: each step streams every weight", "peaks": pk["source"]},
        "e2e": {"value": m4["decode_e2e_tok_s"], "unit": "tok/s"}, "gpu_launches": launches,
        "sizes": sizes, "kernels": kernels, "clocks": clocks}))
    return 0


def design_engine(config: dict, max_seqs: int, tokens_per_seq: int):
    from tandem_b200 import EngineConfig, LLMEngine
    from tandem_b200.engine.core import random_model

    max_len = max(4096, -(-tokens_per_seq // PAGE) * PAGE)
    if "max_position_embeddings" in config:
        config = dict(config, max_position_embeddings=max_len)
    decoder, cfg = random_model(config, seed=0, dtype="bfloat16")
    return LLMEngine(EngineConfig(model="", dtype="bfloat16", block_size=PAGE, num_kv_blocks=max_seqs * (-(-tokens_per_seq // PAGE)) + 8,
                                  max_num_seqs=max_seqs, max_num_batched_tokens=2048, max_model_len=max_len, cuda_graph=True,
                                  cuda_graph_max_bs=max_seqs), decoder=decoder, model_config=cfg, load_tokenizer=False)


def design_prefill_ms(eng, warmup: int, reps: int = 3) -> float:
    import torch

    from tandem_b200.engine.executor import StepEntry

    toks = prompts(1, seed=99)[0]
    times = []
    for i in range(warmup + reps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        eng.executor.step([StepEntry(f"p{i}", toks, [PROMPT - 1])], end=[f"p{i}"])
        stop.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(start.elapsed_time(stop))
    return sorted(times)[len(times) // 2]


def main_design(args) -> int:
    import gc

    import torch

    from tandem_b200.kernels import microbench

    pk = peaks()
    sampler = ClockSampler()
    sampler.start()
    sizes = {}
    launches = 0
    for size, (fum, qwen) in DESIGN_SIZES.items():
        row = {}
        for name, config in (("fumanex", fum), ("qwen3", qwen)):
            eng = design_engine(config, args.batch, PROMPT + NEW_TOKENS + args.steps + 2 * args.warmup + 32)
            d = measure_decode(eng, args.batch, args.steps, args.warmup, PROMPT, NEW_TOKENS)
            ms = design_prefill_ms(eng, args.warmup)
            row[name] = {"prefill_tok_s": round(PROMPT * 1000.0 / ms, 1), "prefill_ms": round(ms, 3), "decode_tok_s": round(d["tok_s"], 1),
                         "decode_ms_per_step": round(d["ms"], 4), "decode_e2e_tok_s": round(d["e2e_tok_s"], 1),
                         "launches_per_decode_step": int(d["launches"]), "parameters": eng.decoder.num_parameters}
            launches += int(d["launches"]) * args.steps
            del eng, d
            gc.collect()
            torch.cuda.empty_cache()
        sizes[size] = row
    with torch.inference_mode():
        att = microbench.sink_attention_case(PROMPT, args.batch, PROMPT, 32, 8, 128, 128, PAGE, 1024, 4, 20, True)
        rec = microbench.recurrence_case(PROMPT, args.batch, 32, 128, 128, 20, True)
    kernels = {
        "sink_attention_tiles_prompt_2048": {"us": round(att["prefill_us"], 1), "tflops": round(att["prefill_tflops"], 1),
                                             "frac_of_bf16_peak": round(att["prefill_tflops"] / pk["tflops"], 4)},
        "sink_attention_decode_b%d" % args.batch: {"us": round(att["decode_us"], 1), "gbs": round(att["decode_gbs"], 1),
                                                   "frac_of_hbm": round(att["decode_gbs"] / pk["hbm_gbs"], 4)},
        "decay_recurrence_prompt_2048": {"us": round(rec["prefill_us"], 1), "tflops_fp32": round(rec["prefill_tflops"], 2)},
        "decay_recurrence_decode_b%d" % args.batch: {"us": round(rec["decode_us"], 1), "gbs": round(rec["decode_gbs"], 1),
                                                     "frac_of_hbm": round(rec["decode_gbs"] / pk["hbm_gbs"], 4)},
    }
    clocks = sampler.stop()
    f4 = sizes["4k"]["fumanex"]
    print(json.dumps({
        "metric": f"decode tok/s at batch {args.batch}, Fumanex (8 layers, width 4096), {PROMPT:,}-token prompts (one B200)",
        "value": f4["decode_tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": f4["decode_ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights and random token ids",
        "config": {"model": "Fumanex beside Qwen3 at equal size", "global_batch": args.batch, "seq_len": PROMPT, "page_size": PAGE,
                   "parallelism": "single GPU", "l2": "inputs larger than L2: each step streams every weight", "peaks": pk["source"]},
        "e2e": {"value": f4["decode_e2e_tok_s"], "unit": "tok/s"}, "gpu_launches": launches,
        "sizes": sizes, "kernels": kernels, "clocks": clocks}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (both numbers are reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--no-extra", action="store_true", help="skip the Qwen3-32B decode and Qwen3-14B mixed-workload figures")
    ap.add_argument("--no-cuda-graph", action="store_true")
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES))
    ap.add_argument("--prompt-len", type=int, default=PROMPT, help="prompt length of the decode measurements")
    ap.add_argument("--new-tokens", type=int, default=None)
    ap.add_argument("--workload", default="decode", choices=["decode", "mixed"])
    ap.add_argument("--policy", default="prefill_first", choices=["prefill_first", "decode_first"])
    ap.add_argument("--design", default=None, choices=["fumanex", "kamelorn", "muzopel", "deletar"], help="another design beside Qwen3 at equal size (a line of its own)")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not measured (use --gpus 1)")
        return 2
    if args.impl == "reference":
        from baseline.reference_arm import run_reference

        print(json.dumps(run_reference(args, SHAPES, prompts, ClockSampler)))
        return 0
    args.warmup = max(3, args.warmup)
    if args.design == "fumanex":
        return main_design(args)
    if args.design == "kamelorn":
        return main_kamelorn(args)
    if args.design == "muzopel":
        return main_muzopel(args)
    if args.design == "deletar":
        return main_deletar(args)
    name, shape = SHAPES[args.shape]
    if args.layers is None:
        args.layers = shape["num_hidden_layers"]
    if args.workload == "mixed":
        args.new_tokens = args.new_tokens or 128
        if args.batch == 8:
            args.batch = 32
        return main_mixed(args, name, shape)
    args.new_tokens = args.new_tokens or NEW_TOKENS

    pk = peaks()
    max_batch = max(args.batch, 1 if args.no_points else 64)
    eng = build_engine(shape, args.layers, max_batch,
                       max(args.prompt_len, PROMPT) + args.new_tokens + args.steps + 2 * args.warmup + 32, not args.no_cuda_graph)
    sampler = ClockSampler()
    sampler.start()
    main_pt = measure_decode(eng, args.batch, args.steps, args.warmup, args.prompt_len, args.new_tokens)
    pre = measure_prefill(eng, args.warmup)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(measure_decode(eng, b, args.steps, args.warmup, args.prompt_len,
                                                          args.new_tokens)["tok_s"], 1)
    clocks = sampler.stop()
    c = eng.model_config
    h2d_bytes = main_pt["h2d"]
    extra = {}
    if not args.no_extra and not args.no_points and args.shape == "8b" and args.layers == shape["num_hidden_layers"]:
        del eng  # the other models get the memory
        extra = measure_extras(min(args.steps, 32), args.warmup)
        graphs_on = not args.no_cuda_graph
    else:
        graphs_on = eng.graphs is not None
    achieved = main_pt["bytes"] / (main_pt["ms"] * 1e-3) / 1e9
    out = {
        "metric": f"decode tok/s at batch {args.batch}, {name}, {args.prompt_len:,}-token prompts (one B200)",
        "value": round(main_pt["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_pt["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights N(0,0.02) and random token ids",
        "config": {"model": name, "layers": c.num_hidden_layers, "layers_full": shape["num_hidden_layers"],
                   "hidden": c.hidden_size, "q_heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
                   "head_dim": c.head_dim, "intermediate": c.intermediate_size, "vocab": c.vocab_size,
                   "global_batch": args.batch, "seq_len": main_pt["context"], "prompt_len": args.prompt_len, "page_size": PAGE,
                   "parallelism": "single GPU", "cuda_graph": graphs_on,
                   "l2": "inputs larger than L2: each step streams every weight", "peaks": pk["source"]},
        "e2e": {"value": round(main_pt["e2e_tok_s"], 1), "unit": "tok/s", "ms_per_step": round(main_pt["e2e_ms"], 4),
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4 * (args.batch + 1)},
        "gpu_launches": int(main_pt["launches"]) * args.steps,
        "prefill": {"value": round(pre["tok_s"], 1), "tokens": PROMPT, "ms": round(pre["ms"], 3),
                    "frac": round(pre["flops"] / (pre["ms"] * 1e-3) / (pk["tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks,
    }
    if extra:
        out["extra"] = extra
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
