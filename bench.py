#!/usr/bin/env python3
"""Benchmark: decode tokens/s and prefill tokens/s for the Qwen2.5-0.5B shape with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

A "step" is one decode step of a batch of requests (default 8) that each hold a prompt of
512 tokens; W untimed warm-up steps, then exactly K timed steps between CUDA events.
`value` is decoded tokens per second with the sampled ids staying on the device (the
reference's --gpu-feedback mode, rust/engine/benches/qwen2.rs:182-229); `e2e` is the same
through the Python entry point `LLM.generate`, with host token ids going in and coming out
every step.  The line also carries a 2,048-token prefill, the decode step's HBM roofline
fraction, decode at batch 1 and 64, the GPU's clocks during the timed region and the number
of this repository's kernel launches inside it.  Inputs are larger than the L2 cache: a
decode step streams about 1 GB of weights, so nothing is flushed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Layer sizes of the Qwen2.5-0.5B shape (random weights, seed 0, N(0, 0.02)).
QWEN25_05B = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=151936, hidden_size=896,
    intermediate_size=4864, num_hidden_layers=24, num_attention_heads=14, num_key_value_heads=2,
    rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=4096, hidden_act="silu",
    tie_word_embeddings=True, use_sliding_window=False, eos_token_id=151645)
# Further sizes of the same architecture (--shape), for measurements beyond the headline configuration.
SHAPES = {
    "0.5B": QWEN25_05B,
    "1.5B": dict(QWEN25_05B, hidden_size=1536, intermediate_size=8960, num_hidden_layers=28, num_attention_heads=12,
                 num_key_value_heads=2, max_position_embeddings=8192),
    "7B": dict(QWEN25_05B, vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
               num_attention_heads=28, num_key_value_heads=4, max_position_embeddings=16384,
               tie_word_embeddings=False),
}
PROMPT_LEN, NEW_TOKENS, PREFILL_TOKENS, PAGE_SIZE = 512, 256, 2048, 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            raw = json.load(open(path))
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"])}, "measured"
        except Exception:  # noqa: BLE001
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "25"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm = [int(r[0]) for r in self.rows if r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def model_folder(cfg_dict, layers):
    """A random-weights model folder for the configuration (made once per machine and size)."""
    import torch
    from llm_inference_lab_b200.registry import resolve
    from llm_inference_lab_b200.weights import write_random_model

    cfg_dict = dict(cfg_dict, num_hidden_layers=layers)
    folder = os.path.join(tempfile.gettempdir(), f"lab_b200_bench_qwen2_H{cfg_dict['hidden_size']}_L{layers}_{os.getuid()}")
    marker = os.path.join(folder, ".complete")
    if not os.path.exists(marker):
        cfg = resolve(cfg_dict).config_class.from_dict(cfg_dict)
        write_random_model(cfg, folder, seed=0, dtype=torch.bfloat16, std=0.02, norm_std=0.0)
        open(marker, "w").write("ok")
    return folder


def decode_bytes(cfg, layers, batch, mean_ctx):
    """Bytes a decode step has to read: every weight once, and the cache of the live requests."""
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    d = h // cfg["num_attention_heads"]
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    per_layer = (nq + 2 * nkv) * d * h + (nq + 2 * nkv) * d + nq * d * h + 3 * h * i + 2 * h
    weights = 2 * (layers * per_layer + v * h + h)   # the head's matrix once (tied or not, a decode step reads one)
    cache = 2 * batch * mean_ctx * layers * 2 * nkv * d
    return weights + cache


def prefill_flops(cfg, layers, tokens):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    d = h // cfg["num_attention_heads"]
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    linear = 2 * tokens * layers * ((nq + 2 * nkv) * d * h + nq * d * h + 3 * h * i) + 2 * v * h
    attention = layers * nq * 2 * 2 * d * tokens * (tokens + 1) // 2
    return linear + attention


def run_decode(engine, graphs, batch, steps, warmup, rng, clocks=None, repeats=1):
    """Prefill `batch` prompts of PROMPT_LEN tokens, then time `steps` decode steps `repeats` times
    (device feedback: the sampled ids stay on the device).  `graphs` None: every step is launched
    kernel by kernel (eager) instead of replayed from a CUDA graph.  Returns a list of
    (ms of the region, launches, mean context length) per repeat."""
    import torch
    from llm_inference_lab_b200.engine import Entry
    from llm_inference_lab_b200.kernels import ops

    ids = list(range(batch))
    vocab = engine.vocab
    first = []
    for r in ids:
        prompt = [int(t) for t in rng.integers(0, vocab, PROMPT_LEN)]
        logits = engine.step([Entry(r, prompt, [PROMPT_LEN - 1])])
        first.append(int(logits.argmax(dim=-1).item()))
    if graphs is not None:
        out = graphs.step(ids, tokens=first)
        step = lambda: graphs.step(ids)  # noqa: E731
    else:
        eager = EagerDecode(engine, ids, first)
        out = eager.step()
        step = eager.step
    for _ in range(max(warmup - 1, 0)):
        out = step()
    torch.cuda.synchronize()
    regions = []
    if clocks is not None:
        clocks.__enter__()
    for _ in range(repeats):
        ctx0 = engine.cache.length(ids[0])
        launches0 = ops.COUNTER.launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            out = step()
        e1.record()
        torch.cuda.synchronize()
        regions.append((e0.elapsed_time(e1), ops.COUNTER.launches - launches0, ctx0 + (steps + 1) / 2.0))
    if clocks is not None:
        clocks.__exit__(None, None, None)
    tokens = out.cpu().tolist()
    assert all(0 <= t < vocab for t in tokens), "decode produced an invalid token"
    ops.take_device_errors()
    for r in ids:
        engine.close(r)
    return regions


class EagerDecode:
    """Decode steps launched kernel by kernel through `Engine.step`, the sampled ids fed forward on
    the device (the host never reads them): the eager twin of the decode graphs, for the figure the
    reference reports beside its graph mode (roadmap.md:653-656)."""

    def __init__(self, engine, ids, first):
        import torch
        self.engine, self.ids = engine, ids
        self.tokens = torch.tensor(first, dtype=torch.int32, device=engine.device)
        self.rows = torch.arange(len(ids), dtype=torch.int32, device=engine.device)

    def step(self):
        from llm_inference_lab_b200.kernels import ops
        eng = self.engine
        pairs = [(r, 1) for r in self.ids]
        began = eng._begin(pairs, False)
        try:
            ctx, _ = eng._pack_pairs(pairs, self.tokens)
            logits = eng.model.forward(ctx, eng.views, self.rows)
            ops.sample(logits, None, None, None, out=self.tokens)
        except Exception:
            eng._fail(began)
            raise
        eng._end(pairs, False)
        return self.tokens


def run_stack_stamps(engine, batch, rng):
    """The decode stack's own clock: CTA 0 stamps every phase (start, first operand built, first item
    done, all items done) and every CTA stamps the end of its share; printed per kind of phase."""
    import numpy as np
    import torch
    from llm_inference_lab_b200.engine import Entry

    stack = engine.model.decode_stack
    if stack is None:
        return {"error": "the model's layers do not fit the decode stack"}
    calls = len(stack.order)
    for r in range(batch):
        engine.step([Entry(r, [int(t) for t in rng.integers(0, engine.vocab, PROMPT_LEN)], [])])
    stack.stamps = torch.zeros((4 * 5 * calls + 1 + 5 * calls * stack.grid,), dtype=torch.int64, device="cuda")
    for _ in range(4):
        engine.step([Entry(r, [5], [0]) for r in range(batch)])
        torch.cuda.synchronize()
    full = stack.stamps.cpu().numpy().astype(np.int64)
    stack.stamps = None
    for r in range(batch):
        engine.close(r)
    t, per = full[: 4 * 5 * calls + 1], full[4 * 5 * calls + 1:].reshape(5 * calls, stack.grid)
    ph = t[:-1].reshape(calls, 5, 4)
    starts = np.concatenate([t[:-1].reshape(-1, 4)[:, 0], t[-1:]])
    out = {"kernel_us": round(float(t[-1] - t[0]) / 1e3, 1), "layer_calls": calls, "batch": batch, "phases": {}}
    skip = min(2, calls - 1)
    for k, name in enumerate(["qkv", "attention", "o_proj", "gate_up", "down"]):
        length = (starts[1:] - starts[:-1]).reshape(calls, 5)[skip:, k]
        entry = {"phase_us": round(float(length.mean()) / 1e3, 2)}
        if k != 1:      # (the warp that stamps takes no part in the attention phase)
            done = (per.reshape(calls, 5, -1)[skip:, k] - ph[skip:, k, 0][:, None]) / 1e3
            entry["cta_done_us_median"] = round(float(np.median(done)), 2)
            entry["cta_done_us_max"] = round(float(done.max(1).mean()), 2)
            entry["cta0_operand_us"] = round(float((ph[skip:, k, 1] - ph[skip:, k, 0]).mean()) / 1e3, 2)
            entry["cta0_item_us"] = round(float((ph[skip:, k, 2] - ph[skip:, k, 1]).mean()) / 1e3, 2)
        out["phases"][name] = entry
    return out


def median_region(regions):
    ordered = sorted(regions, key=lambda r: r[0])
    return ordered[len(ordered) // 2]


def run_prefill(engine, rng, repeats=5):
    import torch
    from llm_inference_lab_b200.engine import Entry

    times = []
    for it in range(3 + repeats):
        prompt = [int(t) for t in rng.integers(0, engine.vocab, PREFILL_TOKENS)]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        logits = engine.step([Entry(1000 + it, prompt, [PREFILL_TOKENS - 1])])
        e1.record()
        torch.cuda.synchronize()
        assert bool(torch.isfinite(logits).all())
        engine.close(1000 + it)
        if it >= 3:
            times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def run_e2e(folder, batch, steps, warmup):
    """Decode tokens/s through LLM.generate: host ids in and out every step."""
    import numpy as np
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.sampling import SamplingConfig

    llm = LLM(folder, "bf16", max_batch_tokens=8192, page_size=PAGE_SIZE,
              kv_tokens=batch * (PROMPT_LEN + NEW_TOKENS + PAGE_SIZE), max_requests=max(batch, 1),
              max_seq_len=4096, cuda_graph=True)
    rng = np.random.default_rng(1)
    prompts = [[int(t) for t in rng.integers(0, llm.engine.vocab, PROMPT_LEN)] for _ in range(batch)]
    n_new = min(NEW_TOKENS, warmup + steps + 2)
    llm.generate(prompts, SamplingConfig(max_new_tokens=4, ignore_eos=True))          # compiles and captures
    llm.step_log.clear()
    results = llm.generate(prompts, SamplingConfig(max_new_tokens=n_new, ignore_eos=True))
    assert all(len(r.tokens) == n_new for r in results)
    decode = [(t, n) for t, n, is_decode, _ in llm.step_log if is_decode and n == batch]
    timed = decode[warmup: warmup + steps + 1]
    k = len(timed) - 1
    seconds = timed[-1][0] - timed[0][0]
    meta_words = llm.graphs.cached[next(iter(llm.graphs.cached))].layout.total
    # Every decode step copies its metadata (positions, cache slots, block tables, lengths) from pinned
    # host memory and its sampled ids back to the host.  The ids themselves go from one step to the
    # next on the device: the step after is launched before the host has read them (lookahead).
    return {"value": batch * k / seconds, "unit": "tokens/s", "steps": k,
            "h2d_bytes_per_step": 4 * meta_words, "d2h_bytes_per_step": 4 * batch,
            "note": "LLM.generate; each step is launched one step ahead of the host's read of the sampled ids"}


def run_serve(folder, cfg, layers, requests, chunk, new_tokens, max_seq, lo=128, hi=2048, graph=True):
    """Continuous batching through LLM.generate: `requests` prompts of lo..hi tokens arrive at once, prompts
    are cut into portions under a budget of `chunk` tokens a step (decoding requests first), and every
    request decodes `new_tokens` tokens.  Timed on the host around the whole call, after two untimed
    runs of the same work (they compile, and capture the graphs the timed run replays)."""
    import numpy as np
    import torch
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.sampling import SamplingConfig

    rng = np.random.default_rng(2)
    lengths = [int(n) for n in rng.integers(lo, hi + 1, requests)]
    need = sum(-(-(n + new_tokens) // PAGE_SIZE) * PAGE_SIZE for n in lengths)
    llm = LLM(folder, "bf16", max_batch_tokens=chunk, page_size=PAGE_SIZE, kv_tokens=need + 64 * PAGE_SIZE,
              max_requests=requests, max_seq_len=max_seq, cuda_graph=graph)
    prompts = [[int(t) for t in rng.integers(0, llm.engine.vocab, n)] for n in lengths]
    sampling = SamplingConfig(max_new_tokens=new_tokens, ignore_eos=True)
    for _ in range(2):      # the second run captures the step shapes that came twice
        llm.generate(prompts, sampling)
    torch.cuda.synchronize()
    llm.step_log.clear()
    steps0 = llm.steps
    replays0 = (llm.graphs.replays if llm.graphs else 0, llm.engine.graph_replays)
    t0 = time.perf_counter()
    results = llm.generate(prompts, sampling)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    assert all(r.finish_reason == "length" and len(r.tokens) == new_tokens for r in results)
    generated = requests * new_tokens
    steps = llm.steps - steps0
    log = llm.step_log
    decode_steps = sum(1 for _, _, is_decode, _ in log if is_decode)
    from_graphs = ((llm.graphs.replays if llm.graphs else 0) - replays0[0]) + (llm.engine.graph_replays - replays0[1])
    # Pure decode steps against the HBM roofline: the bytes each has to read (every weight once and
    # the cache of its requests) over the time between its tokens and the previous step's reaching
    # the host (steps run back to back, one launched ahead).
    nbytes = seconds_decode = 0.0
    for prev, cur in zip(log, log[1:]):
        if cur[2] and prev[2]:
            nbytes += decode_bytes(cfg, layers, 0, 0) + kv_bytes_per_token(cfg, layers) * cur[3]
            seconds_decode += cur[0] - prev[0]
    return {"workload": f"continuous batching: {requests} requests at once, prompts of {lo}..{hi} tokens, "
                        f"{chunk} tokens a step, {new_tokens} new tokens each",
            "seconds": round(seconds, 4), "prompt_tokens": sum(lengths), "generated_tokens": generated,
            "total_tokens_per_s": round((sum(lengths) + generated) / seconds, 1),
            "generated_tokens_per_s": round(generated / seconds, 1),
            "steps": steps, "pure_decode_steps": decode_steps,
            "steps_from_graphs": from_graphs, "eager_share": round(1.0 - from_graphs / max(steps, 1), 4),
            "ms_per_step": round(1e3 * seconds / max(steps, 1), 4),
            "decode_hbm_gbs": round(nbytes / max(seconds_decode, 1e-9) / 1e9, 1),
            "ttft_ms_median": round(1e3 * statistics.median(r.ttft for r in results), 2),
            "preemptions": sum(r.preemptions for r in results)}


# ----------------------------------------------------------------------------------------
# --arch sogulix: the Sogulix design beside Qwen2 at equal layer sizes (random weights)
# ----------------------------------------------------------------------------------------
SOGULIX_SHAPES = {
    # width, feed-forward and vocabulary of the Qwen2.5 shape of the same name; mixers sized alike
    "0.5B": dict(heads=14, dim=64, rot_dim=32, vdim=64, kv_rank=256, q_rank=384, window=1024, decay_rank=64),
    "1.5B": dict(heads=12, dim=96, rot_dim=32, vdim=128, kv_rank=512, q_rank=768, window=2048, decay_rank=96),
}


def sogulix_config(shape, layers):
    q, m = SHAPES[shape], SOGULIX_SHAPES[shape]
    mlp = {"kind": "dense", "ff": q["intermediate_size"]}
    delta = {"type": "general_delta", "mlp": mlp,
             "mixer": {"heads": m["heads"], "dim": m["dim"], "decay_rank": m["decay_rank"]}}
    latent = {"type": "latent_attention", "mlp": mlp,
              "mixer": {"heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
                        "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "mask": {"size": m["window"]},
                        "rot": {"base": 10000.0, "dims": m["rot_dim"]}, "scale": (m["dim"] + m["rot_dim"]) ** -0.5}}
    return {"architecture": "Sogulix", "vocab": q["vocab_size"], "width": q["hidden_size"], "norm": {"eps": 1e-6},
            "residual_mult": 0.5, "logit_softcap": 30.0, "layers": [delta if i % 2 == 0 else latent for i in range(layers)]}


def arch_folder(cfg_dict, tag):
    import torch
    from llm_inference_lab_b200.registry import resolve
    from llm_inference_lab_b200.weights import write_random_model

    folder = os.path.join(tempfile.gettempdir(), f"lab_b200_bench_{tag}_{os.getuid()}")
    marker = os.path.join(folder, ".complete")
    if not os.path.exists(marker):
        cfg = resolve(cfg_dict).config_class.from_dict(cfg_dict)
        write_random_model(cfg, folder, seed=0, dtype=torch.bfloat16, std=0.02, norm_std=0.0)
        open(marker, "w").write("ok")
    return folder


def timed(fn, repeats=7, flush=None):
    """Median milliseconds of fn() between CUDA events, after three warm-up calls; `flush` (a buffer
    larger than L2) is overwritten before every timed call."""
    import torch
    times = []
    for it in range(3 + repeats):
        if flush is not None:
            flush.add_(1)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        if it >= 3:
            times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def model_points(folder, batch, prompt_len, prefill_tokens, decode_steps):
    """Prefill and eager decode throughput of a model folder through `Engine.step`."""
    import numpy as np
    import torch
    from llm_inference_lab_b200.engine import Engine, Entry
    from llm_inference_lab_b200.kernels import ops

    rng = np.random.default_rng(0)
    engine = Engine(folder, "bf16", max_tokens=batch * (prompt_len + 256) + prefill_tokens + 64, page_size=PAGE_SIZE,
                    max_requests=batch + 1, max_batch_tokens=max(prefill_tokens, prompt_len), max_seq_len=4096)
    out = {}
    prompt = [int(t) for t in rng.integers(0, engine.vocab, prefill_tokens)]

    def prefill():
        engine.step([Entry(999, prompt, [prefill_tokens - 1])])
        engine.close(999)

    launches0 = ops.COUNTER.launches
    prefill()
    out["prefill_launches"] = ops.COUNTER.launches - launches0
    ms = timed(prefill, repeats=5)
    out["prefill_ms"], out["prefill_tok_s"] = round(ms, 3), round(prefill_tokens / (ms / 1e3), 1)
    for r in range(batch):
        engine.step([Entry(r, [int(t) for t in rng.integers(0, engine.vocab, prompt_len)], [])])
    entries = [Entry(r, [7 + r], [0]) for r in range(batch)]
    launches0 = ops.COUNTER.launches
    engine.step(entries)
    out["decode_launches"] = ops.COUNTER.launches - launches0

    def decode():
        for _ in range(decode_steps):
            engine.step(entries)

    ms = timed(decode, repeats=3) / decode_steps
    out["decode_ms_per_step"], out["decode_tok_s"] = round(ms, 4), round(batch / (ms / 1e3), 1)
    ops.take_device_errors()
    for r in range(batch):
        engine.close(r)
    if engine.decode_graph_capable:
        # the same steps replayed from CUDA graphs, the picked ids fed forward on the device
        from llm_inference_lab_b200.engine.decode_graph import DecodeGraphs
        gms, launches, _ = median_region(run_decode(engine, DecodeGraphs(engine), batch, decode_steps, 5, rng, repeats=3))
        out["decode_graph_ms_per_step"] = round(gms / decode_steps, 4)
        out["decode_graph_tok_s"] = round(batch * decode_steps / (gms / 1e3), 1)
        out["decode_graph_launches_per_step"] = launches // decode_steps
    del engine
    torch.cuda.empty_cache()
    return out


def bench_ctx(q_lens, pos0, page_size, device):
    """A step's context with pages in order, for timing single kernels."""
    import numpy as np
    import torch
    from llm_inference_lab_b200.parts.base import GroupView, StepContext

    kv = [p + n for p, n in zip(pos0, q_lens)]
    blocks = [-(-k // page_size) for k in kv]
    width = (max(blocks) + 7) & ~7
    table = -np.ones((len(q_lens), width), dtype=np.int32)
    at = 0
    for r, b in enumerate(blocks):
        table[r, :b] = np.arange(at, at + b)
        at += b
    row_req = np.concatenate([np.full(n, r) for r, n in enumerate(q_lens)])
    row_pos = np.concatenate([np.arange(p, p + n) for p, n in zip(pos0, q_lens)])
    row_slot = table[row_req, row_pos // page_size] * page_size + row_pos % page_size
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(device)  # noqa: E731
    group = GroupView(page_size, 0, t(row_slot), t(table))
    ctx = StepContext(dtype=torch.bfloat16, device=device, n_tokens=sum(q_lens), n_requests=len(q_lens),
                      token_ids=t(np.zeros(sum(q_lens))), row_req=t(row_req), row_pos=t(row_pos),
                      q_start=t(np.concatenate([[0], np.cumsum(q_lens)])), kv_len=t(kv), pos0=t(pos0),
                      state_slot=t(np.arange(len(q_lens))), groups=[group], q_lens=list(q_lens), kv_lens=kv,
                      state_slots=list(range(len(q_lens))), max_q_len=max(q_lens), max_kv_len=max(kv))
    return ctx, at


def kernel_points(shape, batch, ctx_len, prefill_tokens, pk):
    """The new design's own kernels and Qwen2's like kernels at the shape's sizes, each alone between
    CUDA events with L2 flushed: milliseconds, and the fraction of the roofline (measured copy bandwidth
    for kernels that stream, measured bf16 product rate for the attention kernels of a prompt)."""
    import torch
    from llm_inference_lab_b200.kernels import ops

    dev = torch.device("cuda:0")
    q, m = SHAPES[shape], SOGULIX_SHAPES[shape]
    width, H, D, R, C, V = q["hidden_size"], m["heads"], m["dim"], m["rot_dim"], m["kv_rank"], m["vdim"]
    hd = H * D
    flush = torch.zeros((160 << 20,), dtype=torch.int16, device=dev)
    bw, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    rows = {}

    def record(name, ms, nbytes=None, flops=None):
        entry = {"ms": round(ms, 4)}
        if nbytes is not None:
            entry.update(gbs=round(nbytes / (ms / 1e3) / 1e9, 1), frac_hbm=round(nbytes / (ms / 1e3) / bw, 4))
        if flops is not None:
            entry.update(tflops=round(flops / (ms / 1e3) / 1e12, 2), frac_bf16=round(flops / (ms / 1e3) / tf, 4))
        rows[name] = entry

    bf = lambda *s: torch.randn(*s, device=dev).to(torch.bfloat16)  # noqa: E731
    for label, q_lens, pos0 in (("prefill", [prefill_tokens], [0]), ("decode", [1] * batch, [ctx_len] * batch)):
        T, B = sum(q_lens), len(q_lens)
        ctx, pages = bench_ctx(q_lens, pos0, PAGE_SIZE, dev)
        # generalized delta rule: reads five 32-bit projections and the decay's, the state in and out
        proj, dpre = torch.randn(T, 5 * hd + 64, device=dev), torch.randn(T, hd, device=dev)
        state = torch.zeros(B, H, D, D, device=dev)
        ones = bf(hd)
        ms = timed(lambda: ops.delta_rule(proj, dpre, ones, ones, ones, state, ctx, H, D, 1e-6, 0.6), flush=flush)
        record(f"delta_rule {label}", ms, nbytes=T * hd * (6 * 4 + 2) + 2 * state.numel() * 4,
               flops=None if label == "decode" else 8.0 * T * H * D * D)
        # latent attention: reads the window's latents once per request (decode) or the scores' and the
        # weighted sums' arithmetic (prompt)
        W = C + R
        cache = bf(pages, PAGE_SIZE, W)
        q_cat = torch.randn(T, H, W, device=dev)
        sink = torch.zeros(H, device=dev)
        keys = [min(m["window"], p + n) for p, n in zip(pos0, q_lens)]
        pairs = sum(sum(min(m["window"], p + i + 1) for i in range(n)) for p, n in zip(pos0, q_lens))
        if label == "decode":
            # single tokens read the latents as they are cached (absorbed form)
            ms = timed(lambda: ops.latent_attention(q_cat, cache, sink, ctx, ctx.groups[0], H, C, m["window"], 0.1),
                       flush=flush)
            record("latent_attention decode", ms, nbytes=sum(keys) * W * 2 + T * H * (W * 4 + C * 2),
                   flops=2.0 * pairs * H * (W + C))
        elif ops.latent_plain_form_supported(torch.bfloat16, D, R, V):
            # prompts: keys and values projected up for the step, then the tensor-core attention kernel
            hsz = ops.latent_head_size(D, R, V)
            qp, outp, w_up = bf(T, H * hsz), torch.empty(T, H * hsz, dtype=torch.bfloat16, device=dev), bf(H * (D + V), C)
            ms = timed(lambda: ops.latent_attention_plain_form(qp, cache, w_up, sink, ctx, ctx.groups[0], H, D, R, V, C,
                                                               m["window"], 0.1, 16, outp), flush=flush)
            record("latent_attention prefill (gather, project up, scatter, attention)", ms,
                   flops=2.0 * sum(keys) * C * H * (D + V) + 4.0 * pairs * H * hsz)
        # Qwen2's attention at the same heads (grouped 7:1 as in the shape) and head size
        nq, nkv = q["num_attention_heads"], q["num_key_value_heads"]
        d = q["hidden_size"] // nq
        if ops.attention_tc_supported(d):
            ck, cv = bf(pages, nkv, PAGE_SIZE, d), bf(pages, nkv, PAGE_SIZE, d)
            qq = bf(T, nq * d)
            ms = timed(lambda: ops.attention_tc(qq, ck, cv, ctx.q_start, ctx.kv_len, ctx.pos0, ctx.groups[0].block_table,
                                                B, ctx.q_lens, ctx.max_kv_len, nq, nkv, d, 0, d ** -0.5), flush=flush)
            all_pairs = sum(sum(p + i + 1 for i in range(n)) for p, n in zip(pos0, q_lens))
            record(f"qwen2 attention {label}", ms, nbytes=sum(p + n for p, n in zip(pos0, q_lens)) * 2 * nkv * d * 2
                   + 2 * T * nq * d * 2, flops=4.0 * all_pairs * nq * d)
        # the row-wise operators around a block
        x = torch.randn(T, width, device=dev)
        w1 = bf(width)
        kept = torch.zeros(B, width, device=dev)

        def norms():
            n, _ = ops.norm_stream(x, 1e-6, 1.0, weight_f32=w1, weight=w1)
            ops.token_shift(n, w1, kept, ctx)

        ms = timed(norms, flush=flush)
        record(f"two norms + token shift {label}", ms, nbytes=T * width * (4 + 4 + 2 + 4 + 2))
        a, f = torch.randn(T, width, device=dev), torch.randn(T, width, device=dev)
        ms = timed(lambda: ops.stream_add(x, a, w1, f, w1, 0.5), flush=flush)
        record(f"stream add {label}", ms, nbytes=T * width * 16)
        xb, delta = bf(T, width), bf(T, width)
        ms = timed(lambda: ops.add_rmsnorm(xb, w1, 1e-6, delta=delta), flush=flush)
        record(f"qwen2 add + norm {label}", ms, nbytes=T * width * 8)
    ops.take_device_errors()
    return rows


def run_arch_sogulix(args):
    shape, layers = args.shape, args.layers or 4
    pk, pk_src = peaks()
    qcfg = dict(SHAPES[shape], num_hidden_layers=layers)
    folders = {"sogulix": arch_folder(sogulix_config(shape, layers), f"sogulix_{shape}_L{layers}"),
               "qwen2": model_folder(SHAPES[shape], layers)}
    clocks = ClockSampler()
    with clocks:
        models = {name: model_points(folder, args.batch, args.prompt_len, PREFILL_TOKENS, 20)
                  for name, folder in folders.items()}
        kernels = kernel_points(shape, args.batch, args.prompt_len + 512, PREFILL_TOKENS, pk)
    print(json.dumps({
        "arch": "sogulix", "beside": "qwen2", "shape": shape, "layers": layers, "batch": args.batch,
        "prompt_len": args.prompt_len, "prefill_tokens": PREFILL_TOKENS, "dtype": "bf16", "mode": "eager launches",
        "data": "synthetic: random weights N(0, 0.02) seed 0", "sogulix_mixers": SOGULIX_SHAPES[shape],
        "hidden": qcfg["hidden_size"], "intermediate": qcfg["intermediate_size"], "vocab": qcfg["vocab_size"],
        "models": models, "kernels": kernels, "peaks": dict(pk, source=pk_src), "clocks": clocks.summary()}))
    return 0


# ----------------------------------------------------------------------------------------
# --arch ritizen: the Ritizen design beside Sogulix and Qwen2 at equal layer sizes (random weights)
# ----------------------------------------------------------------------------------------
RITIZEN_SHAPES = {
    # width, feed-forward and vocabulary of the Qwen2.5 shape of the same name; attention heads as there;
    # the recurrent mixers sized like the attention (state-space: inner = 2 x width)
    "0.5B": dict(heads=14, kv_heads=2, dim=64, vdim=64, chunk=1024, lin_heads=14, lin_dim=64, lin_vdim=64,
                 ssm_heads=28, ssm_vdim=64, ssm_state=64, ssm_groups=2, taps=4, norm_groups=2),
    "1.5B": dict(heads=12, kv_heads=2, dim=128, vdim=128, chunk=2048, lin_heads=12, lin_dim=128, lin_vdim=128,
                 ssm_heads=24, ssm_vdim=128, ssm_state=128, ssm_groups=2, taps=4, norm_groups=2),
}


def ritizen_config(shape, layers):
    """Layers in the order attention, attention on the first one's keys and values, state-space, side by side."""
    q, m = SHAPES[shape], RITIZEN_SHAPES[shape]
    mlp = {"kind": "dense", "ff": q["intermediate_size"]}
    att = {"heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"], "scale": m["dim"] ** -0.5}
    decay = [1.0 - 2.0 ** -(2 + 6 * h / max(1, m["lin_heads"] - 1)) for h in range(m["lin_heads"])]
    kinds = [
        lambda i: {"type": "attention", "mixer": dict(att), "mlp": mlp},
        lambda i: {"type": "attention", "mixer": dict(att, kv_from=i - 1), "mlp": mlp},
        lambda i: {"type": "mamba2", "mlp": None,
                   "mixer": {"heads": m["ssm_heads"], "vdim": m["ssm_vdim"], "state": m["ssm_state"],
                             "groups": m["ssm_groups"], "conv": m["taps"], "norm_groups": m["norm_groups"]}},
        lambda i: {"type": "parallel", "mlp": mlp,
                   "mixer": {"left": dict(att, mask={"size": m["chunk"]}), "left_scale": 0.6, "right_scale": 1.1,
                             "right": {"heads": m["lin_heads"], "dim": m["lin_dim"], "vdim": m["lin_vdim"],
                                       "decay": decay}}},
    ]
    return {"architecture": "Ritizen", "vocab": q["vocab_size"], "width": q["hidden_size"], "max_positions": 4096,
            "norm": {"eps": 1e-6}, "layers": [kinds[i % 4](i) for i in range(layers)]}


def kernel_points_ritizen(shape, batch, ctx_len, prefill_tokens, pk):
    """The Ritizen design's own kernels beside the like kernels of Sogulix (the recurrence, the stream's sum)
    and of Qwen2 (attention, the rotation with its cache write, add + norm) at the shape's sizes, each alone
    between CUDA events with L2 flushed: milliseconds and the fraction of the roofline (measured copy bandwidth
    for kernels that stream, measured bf16 product rate for the attention kernels of a prompt)."""
    import torch
    from llm_inference_lab_b200.kernels import ops

    dev = torch.device("cuda:0")
    q, m, sg = SHAPES[shape], RITIZEN_SHAPES[shape], SOGULIX_SHAPES[shape]
    width = q["hidden_size"]
    flush = torch.zeros((160 << 20,), dtype=torch.int16, device=dev)
    bw, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    rows = {}

    def record(name, ms, nbytes=None, flops=None):
        entry = {"ms": round(ms, 4)}
        if nbytes is not None:
            entry.update(gbs=round(nbytes / (ms / 1e3) / 1e9, 1), frac_hbm=round(nbytes / (ms / 1e3) / bw, 4))
        if flops is not None:
            entry.update(tflops=round(flops / (ms / 1e3) / 1e12, 2), frac_bf16=round(flops / (ms / 1e3) / tf, 4))
        rows[name] = entry

    bf = lambda *s: torch.randn(*s, device=dev).to(torch.bfloat16)  # noqa: E731
    f32 = lambda *s: torch.randn(*s, device=dev)  # noqa: E731
    for label, q_lens, pos0 in (("prefill", [prefill_tokens], [0]), ("decode", [1] * batch, [ctx_len] * batch)):
        T, B = sum(q_lens), len(q_lens)
        ctx, pages = bench_ctx(q_lens, pos0, PAGE_SIZE, dev)
        # the recurrence with a fixed decay per head: reads q, k, v (32-bit), writes o, the state in and out
        H, N, V = m["lin_heads"], m["lin_dim"], m["lin_vdim"]
        proj = f32(T, 2 * H * N + 2 * H * V)
        state = torch.zeros(B, H, N, V, device=dev)
        decay = torch.full((H,), 0.97, device=dev)
        ms = timed(lambda: ops.decay_scan(proj[:, : H * N], proj[:, H * N: 2 * H * N], proj[:, 2 * H * N: 2 * H * N + H * V],
                                          state, ctx, H, H, N, V, a_head=decay, silu=True), flush=flush)
        record(f"decay_scan fixed decay {label}", ms, nbytes=T * (2 * H * N + 2 * H * V) * 4 + 2 * state.numel() * 4,
               flops=None if label == "decode" else 4.0 * T * H * N * V)
        # the same recurrence with a decay and a key scale per token (state-space), q and k shared by groups
        H2, N2, V2, G2 = m["ssm_heads"], m["ssm_state"], m["ssm_vdim"], m["ssm_groups"]
        conv = f32(T, H2 * V2 + 2 * G2 * N2)
        a_tok, s_tok = torch.rand(T, H2, device=dev), torch.rand(T, H2, device=dev)
        state2 = torch.zeros(B, H2, N2, V2, device=dev)
        ms = timed(lambda: ops.decay_scan(conv[:, H2 * V2 + G2 * N2:], conv[:, H2 * V2: H2 * V2 + G2 * N2], conv[:, : H2 * V2],
                                          state2, ctx, H2, G2, N2, V2, a_tok=a_tok, s_tok=s_tok), flush=flush)
        record(f"decay_scan decay per token {label}", ms,
               nbytes=T * (2 * G2 * N2 + 2 * H2 * V2 + 2 * H2) * 4 + 2 * state2.numel() * 4,
               flops=None if label == "decode" else 4.0 * T * H2 * N2 * V2)
        # Sogulix's recurrence (the generalized delta rule) at its shape of the same name
        Hs, Ds = sg["heads"], sg["dim"]
        sproj, dpre = f32(T, 5 * Hs * Ds + 64), f32(T, Hs * Ds)
        sstate = torch.zeros(B, Hs, Ds, Ds, device=dev)
        ones = bf(Hs * Ds)
        ms = timed(lambda: ops.delta_rule(sproj, dpre, ones, ones, ones, sstate, ctx, Hs, Ds, 1e-6, 0.6), flush=flush)
        record(f"sogulix delta_rule {label}", ms, nbytes=T * Hs * Ds * (6 * 4 + 2) + 2 * sstate.numel() * 4,
               flops=None if label == "decode" else 8.0 * T * Hs * Ds * Ds)
        # the state-space mixer's preparation and the gate + norm that close both recurrent mixers
        inner, gn = H2 * V2, G2 * N2
        sproj2 = f32(T, 2 * inner + 2 * gn + H2)
        kept = torch.zeros(B, m["taps"] - 1, inner + 2 * gn, device=dev)
        tw, tb, hb = bf(inner + 2 * gn, m["taps"]), bf(inner + 2 * gn), bf(H2)
        ms = timed(lambda: ops.ssm_prepare(sproj2, inner, 2 * inner + 2 * gn, inner + 2 * gn, m["taps"], H2, tw, tb, hb, hb,
                                           kept, ctx), flush=flush)
        record(f"ssm_prepare {label}", ms, nbytes=T * ((inner + 2 * gn + H2) * 4 + (inner + 2 * gn + 2 * H2) * 4))
        o, wn = f32(T, inner), bf(inner)
        ms = timed(lambda: ops.gated_norm(o, sproj2[:, :inner], wn, 1e-6, parts=m["norm_groups"], gate_first=True, skip=hb,
                                          x=conv[:, :inner], head_size=V2), flush=flush)
        record(f"gated_norm {label}", ms, nbytes=T * inner * (4 + 4 + 4 + 2))
        # attention: norms over the whole projections with the paged store, the kernels with a chunk mask, the gate
        nq, nkv, D, Vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        hd = ops.padded_head(D, Vd)
        ck, cv = bf(pages, nkv, PAGE_SIZE, hd), bf(pages, nkv, PAGE_SIZE, hd)
        wide = nq * D + nkv * (D + Vd) + nq * Vd
        aproj = f32(T, wide)
        ab, wq, wk = bf(nq * D + nkv * (D + Vd)), bf(nq * D), bf(nkv * D)
        ms = timed(lambda: ops.qk_norm_store(aproj, ab, wq, wk, ctx.groups[0].row_slot, ck, cv, nq, nkv, D, Vd, hd, 1e-6),
                   flush=flush)
        record(f"qk_norm_store {label}", ms, nbytes=T * ((nq * D + nkv * (D + Vd)) * 4 + (nq + 2 * nkv) * hd * 2))
        qq = bf(T, nq * hd)
        all_pairs = sum(sum(p + i + 1 for i in range(n)) for p, n in zip(pos0, q_lens))
        chunk = m["chunk"]
        in_chunk = sum(sum((p + i) % chunk + 1 for i in range(n)) for p, n in zip(pos0, q_lens))
        for name, ch, pairs, keys in (("causal", 0, all_pairs, sum(p + n for p, n in zip(pos0, q_lens))),
                                      ("chunked", chunk, in_chunk,
                                       sum(min(p + n, (p + n - 1) % chunk + n) for p, n in zip(pos0, q_lens)))):
            ms = timed(lambda: ops.attention(qq, ck, cv, ctx, ctx.groups[0], nq, nkv, hd, 0, D ** -0.5, chunk=ch), flush=flush)
            record(f"attention {name} {label}", ms, nbytes=keys * 2 * nkv * hd * 2 + 2 * T * nq * hd * 2,
                   flops=4.0 * pairs * nq * hd)
        attn = bf(T, nq * hd)
        ms = timed(lambda: ops.head_gate(attn, aproj, nq * D + nkv * (D + Vd), False, nq, Vd, hd), flush=flush)
        record(f"head_gate {label}", ms, nbytes=T * nq * Vd * (2 + 4 + 2))
        # Qwen2's rotation with its cache write, at the same heads
        d = q["hidden_size"] // q["num_attention_heads"]
        qn, qkvh = q["num_attention_heads"], q["num_key_value_heads"]
        if ops.attention_tc_supported(d):
            qkv = bf(T, (qn + 2 * qkvh) * d)
            ck2, cv2 = bf(pages, qkvh, PAGE_SIZE, d), bf(pages, qkvh, PAGE_SIZE, d)
            inv = torch.rand(d // 2, device=dev)
            ms = timed(lambda: ops.rope_kv_write(qkv, ctx.row_pos, inv, d, ctx.groups[0].row_slot, ck2, cv2, qn, qkvh, d),
                       flush=flush)
            record(f"qwen2 rotation + cache write {label}", ms, nbytes=T * (qn + 2 * qkvh) * d * 2 * 2)
        # the sum that closes a sublayer: x += norm(product), with the rounded copy
        x, a, w1 = f32(T, width), f32(T, width), bf(width)
        ms = timed(lambda: ops.stream_norm_add(x, a, w1, 1e-6, copy=True), flush=flush)
        record(f"stream_norm_add {label}", ms, nbytes=T * width * (4 + 4 + 4 + 2))
        fsum = f32(T, width)
        ms = timed(lambda: ops.stream_add(x, a, w1, fsum, w1, 0.5), flush=flush)
        record(f"sogulix stream add {label}", ms, nbytes=T * width * 16)
        xb, delta = bf(T, width), bf(T, width)
        ms = timed(lambda: ops.add_rmsnorm(xb, w1, 1e-6, delta=delta), flush=flush)
        record(f"qwen2 add + norm {label}", ms, nbytes=T * width * 8)
    ops.take_device_errors()
    return rows


def run_arch_ritizen(args):
    shape, layers = args.shape, args.layers or 4
    pk, pk_src = peaks()
    qcfg = dict(SHAPES[shape], num_hidden_layers=layers)
    folders = {"ritizen": arch_folder(ritizen_config(shape, layers), f"ritizen_{shape}_L{layers}"),
               "sogulix": arch_folder(sogulix_config(shape, layers), f"sogulix_{shape}_L{layers}"),
               "qwen2": model_folder(SHAPES[shape], layers)}
    clocks = ClockSampler()
    with clocks:
        models = {name: model_points(folder, args.batch, args.prompt_len, PREFILL_TOKENS, 20)
                  for name, folder in folders.items()}
        kernels = kernel_points_ritizen(shape, args.batch, args.prompt_len + 512, PREFILL_TOKENS, pk)
    print(json.dumps({
        "arch": "ritizen", "beside": ["sogulix", "qwen2"], "shape": shape, "layers": layers, "batch": args.batch,
        "prompt_len": args.prompt_len, "prefill_tokens": PREFILL_TOKENS, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02) seed 0", "ritizen_mixers": RITIZEN_SHAPES[shape],
        "hidden": qcfg["hidden_size"], "intermediate": qcfg["intermediate_size"], "vocab": qcfg["vocab_size"],
        "models": models, "kernels": kernels, "peaks": dict(pk, source=pk_src), "clocks": clocks.summary()}))
    return 0


# ----------------------------------------------------------------------------------------
# --arch bukatar: the Bukatar design beside Ritizen and Qwen2 at equal layer sizes (random weights)
# ----------------------------------------------------------------------------------------
BUKATAR_SHAPES = {
    # width, feed-forward and vocabulary of the Qwen2.5 shape of the same name; attention heads as there; the
    # state-space mixer with inner = 2 x width; experts sized so that a token's share (top experts and the
    # shared one) has the dense feed-forward's rows
    "0.5B": dict(heads=14, kv_heads=2, dim=64, window=1024, keep_first=64, lat_dim=64, lat_rot=32, lat_vdim=64,
                 kv_rank=256, inner=1792, state=16, dt_rank=56, taps=4, experts=8, top=2, expert_ff=1536,
                 shared_ff=1792),
    "1.5B": dict(heads=12, kv_heads=2, dim=128, window=2048, keep_first=128, lat_dim=96, lat_rot=32, lat_vdim=128,
                 kv_rank=512, inner=3072, state=16, dt_rank=96, taps=4, experts=8, top=2, expert_ff=2816,
                 shared_ff=3328),
}


def bukatar_config(shape, layers):
    """Layers in the order state-space, windowed attention, latent attention, latent attention on the third one's
    latents; dense and routed feed-forwards alternate."""
    q, m = SHAPES[shape], BUKATAR_SHAPES[shape]
    dense = {"kind": "dense", "ff": q["intermediate_size"]}
    moe = {"kind": "moe", "router": {"experts": m["experts"], "top": m["top"]}, "expert": {"ff": m["expert_ff"]},
           "shared": {"ff": m["shared_ff"]}}
    lat = {"heads": m["heads"], "dim": m["lat_dim"], "rot_dim": m["lat_rot"], "vdim": m["lat_vdim"],
           "kv_rank": m["kv_rank"], "scale": (m["lat_dim"] + m["lat_rot"]) ** -0.5,
           "rot": {"base": 10000.0, "dims": m["lat_rot"]}}
    kinds = [
        lambda i: {"type": "mamba1", "mlp": dense,
                   "mixer": {"inner": m["inner"], "state": m["state"], "dt_rank": m["dt_rank"], "conv": m["taps"]}},
        lambda i: {"type": "attention", "mlp": moe,
                   "mixer": {"heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["dim"],
                             "scale": m["dim"] ** -0.5, "rot": {"base": 10000.0, "dims": m["dim"] // 2},
                             "mask": {"size": m["window"], "keep_first": m["keep_first"]}}},
        lambda i: {"type": "latent_attention", "mlp": dense, "mixer": dict(lat)},
        lambda i: {"type": "latent_attention", "mlp": moe, "mixer": dict(lat, kv_from=i - 1)},
    ]
    return {"architecture": "Bukatar", "vocab": q["vocab_size"], "width": q["hidden_size"], "norm": {"eps": 1e-6},
            "max_positions": 4096, "layers": [kinds[i % 4](i) for i in range(layers)]}


def kernel_points_bukatar(shape, batch, ctx_len, prefill_tokens, pk):
    """The Bukatar design's own kernels beside the like kernels of Ritizen (the state-space walk and its
    preparation, the attention's store, the sum that closes a sublayer) and of Qwen2 (attention, the gated
    feed-forward's products) at the shape's sizes, each alone between CUDA events with L2 flushed:
    milliseconds and the fraction of the roofline (measured copy bandwidth for kernels that stream, measured
    bf16 product rate for the attention kernels and the products of a prompt)."""
    import torch
    from llm_inference_lab_b200.kernels import ops

    dev = torch.device("cuda:0")
    q, m, rz = SHAPES[shape], BUKATAR_SHAPES[shape], RITIZEN_SHAPES[shape]
    width, ff = q["hidden_size"], q["intermediate_size"]
    flush = torch.zeros((160 << 20,), dtype=torch.int16, device=dev)
    bw, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    rows = {}

    def record(name, ms, nbytes=None, flops=None):
        entry = {"ms": round(ms, 4)}
        if nbytes is not None:
            entry.update(gbs=round(nbytes / (ms / 1e3) / 1e9, 1), frac_hbm=round(nbytes / (ms / 1e3) / bw, 4))
        if flops is not None:
            entry.update(tflops=round(flops / (ms / 1e3) / 1e12, 2), frac_bf16=round(flops / (ms / 1e3) / tf, 4))
        rows[name] = entry

    bf = lambda *s: (0.5 * torch.randn(*s, device=dev)).to(torch.bfloat16)  # noqa: E731
    f32 = lambda *s: 0.5 * torch.randn(*s, device=dev)  # noqa: E731
    for label, q_lens, pos0 in (("prefill", [prefill_tokens], [0]), ("decode", [1] * batch, [ctx_len] * batch)):
        T, B = sum(q_lens), len(q_lens)
        ctx, pages = bench_ctx(q_lens, pos0, PAGE_SIZE, dev)
        # ---- the state-space mixer: convolution + SiLU, then the walk with a decay per channel and state entry
        inner, N, taps = m["inner"], m["state"], m["taps"]
        proj = f32(T, 2 * inner)
        kept = torch.zeros(B, taps - 1, inner, device=dev)
        cw, cb = bf(inner, taps), bf(inner)
        ms = timed(lambda: ops.conv_silu(proj, 0, inner, taps, cw, cb, kept, ctx), flush=flush)
        record(f"conv_silu {label}", ms, nbytes=T * inner * (4 + 4 + 2) + 2 * kept.numel() * 4)
        x32, dt_pre, bc = f32(T, inner), f32(T, inner), f32(T, 2 * N)
        a_log, skip, dtb = bf(inner, N), bf(inner), bf(inner)
        state = torch.zeros(B, inner, N, device=dev)
        ms = timed(lambda: ops.selective_scan(x32, dt_pre, bc, 0, N, proj[:, inner:], a_log, skip, dtb, state, ctx),
                   flush=flush)
        record(f"selective_scan {label}", ms, nbytes=T * (3 * inner * 4 + 2 * N * 4 + inner * 2) + 2 * state.numel() * 4,
               flops=None if label == "decode" else 6.0 * T * inner * N)
        # Ritizen's state-space walk (a decay per head and token) and its preparation, at its shape of the same name
        H2, N2, V2, G2 = rz["ssm_heads"], rz["ssm_state"], rz["ssm_vdim"], rz["ssm_groups"]
        conv = f32(T, H2 * V2 + 2 * G2 * N2)
        a_tok, s_tok = torch.rand(T, H2, device=dev), torch.rand(T, H2, device=dev)
        state2 = torch.zeros(B, H2, N2, V2, device=dev)
        ms = timed(lambda: ops.decay_scan(conv[:, H2 * V2 + G2 * N2:], conv[:, H2 * V2: H2 * V2 + G2 * N2], conv[:, : H2 * V2],
                                          state2, ctx, H2, G2, N2, V2, a_tok=a_tok, s_tok=s_tok), flush=flush)
        record(f"ritizen decay_scan decay per token {label}", ms,
               nbytes=T * (2 * G2 * N2 + 2 * H2 * V2 + 2 * H2) * 4 + 2 * state2.numel() * 4,
               flops=None if label == "decode" else 4.0 * T * H2 * N2 * V2)
        inner2, gn = H2 * V2, G2 * N2
        sproj2 = f32(T, 2 * inner2 + 2 * gn + H2)
        kept2 = torch.zeros(B, rz["taps"] - 1, inner2 + 2 * gn, device=dev)
        tw, tb, hb = bf(inner2 + 2 * gn, rz["taps"]), bf(inner2 + 2 * gn), bf(H2)
        ms = timed(lambda: ops.ssm_prepare(sproj2, inner2, 2 * inner2 + 2 * gn, inner2 + 2 * gn, rz["taps"], H2, tw, tb, hb,
                                           hb, kept2, ctx), flush=flush)
        record(f"ritizen ssm_prepare {label}", ms,
               nbytes=T * ((inner2 + 2 * gn + H2) * 4 + (inner2 + 2 * gn + 2 * H2) * 4))
        # ---- attention: bias + rotation of pairs + paged store, then the kernels with a window, kept first
        # tokens and the denominator's extra one, beside plain causal attention over the same pages
        nq, nkv, D = m["heads"], m["kv_heads"], m["dim"]
        hd = ops.padded_head(D, D)
        ck, cv = bf(pages, nkv, PAGE_SIZE, hd), bf(pages, nkv, PAGE_SIZE, hd)
        aproj, ab = f32(T, (nq + nkv) * D), bf((nq + nkv) * D)
        inv = torch.rand(D // 4, device=dev)
        ms = timed(lambda: ops.rope_pairs_store(aproj, ab, ctx.row_pos, inv, D // 2, ctx.groups[0].row_slot, ck, cv, nq, nkv,
                                                D, D, hd, nq * D, nq * D, torch.bfloat16), flush=flush)
        record(f"rope_pairs_store {label}", ms, nbytes=T * ((nq + nkv) * D * 4 + (nq + 2 * nkv) * hd * 2))
        wq, wk = bf(nq * D), bf(nkv * D)
        aproj3, ab3 = f32(T, (nq + 2 * nkv) * D), bf((nq + 2 * nkv) * D)
        ms = timed(lambda: ops.qk_norm_store(aproj3, ab3, wq, wk, ctx.groups[0].row_slot, ck, cv, nq, nkv, D, D, hd, 1e-6),
                   flush=flush)
        record(f"ritizen qk_norm_store {label}", ms, nbytes=T * ((nq + 2 * nkv) * D * 4 + (nq + 2 * nkv) * hd * 2))
        qq = bf(T, nq * hd)
        win, keep = m["window"], m["keep_first"]

        def seen(pos):            # keys position `pos` sees through the window with kept first tokens
            return min(pos + 1, win) + min(keep, max(0, pos + 1 - win))

        all_pairs = sum(sum(p + i + 1 for i in range(n)) for p, n in zip(pos0, q_lens))
        win_pairs = sum(sum(seen(p + i) for i in range(n)) for p, n in zip(pos0, q_lens))
        win_keys = sum(min(p + n, win + n - 1 + keep) for p, n in zip(pos0, q_lens))
        for name, kw, pairs, keys in (("causal", {}, all_pairs, sum(p + n for p, n in zip(pos0, q_lens))),
                                      ("window + kept + one", dict(keep_first=keep, sink_one=True), win_pairs, win_keys)):
            w_arg = win if kw else 0
            ms = timed(lambda: ops.attention(qq, ck, cv, ctx, ctx.groups[0], nq, nkv, hd, w_arg, D ** -0.5, **kw), flush=flush)
            record(f"attention {name} {label}", ms, nbytes=keys * 2 * nkv * hd * 2 + 2 * T * nq * hd * 2,
                   flops=4.0 * pairs * nq * hd)
        # ---- the feed-forwards: relu squared in the product's epilogue beside the gated product; the routed
        # experts' kernels (pick, layout, grouped products, weighted sum) beside the dense products of equal rows
        xb = bf(T, width)
        w_up, w_gu, w_down = bf(ff, width), bf(2 * ff, width), bf(width, ff)
        ms = timed(lambda: ops.linear(xb, w_up, None, act="relu2"), flush=flush)
        record(f"product + relu squared {label}", ms, nbytes=(ff * width + T * (width + ff)) * 2, flops=2.0 * T * ff * width)
        ms = timed(lambda: ops.linear_gated(xb, w_gu), flush=flush)
        record(f"qwen2 gated product {label}", ms, nbytes=(2 * ff * width + T * (width + ff)) * 2,
               flops=4.0 * T * ff * width)
        hidden = bf(T, ff)
        ms = timed(lambda: ops.linear(hidden, w_down, None, out_f32=True), flush=flush)
        record(f"qwen2 down product {label}", ms, nbytes=(ff * width + T * ff) * 2 + T * width * 4, flops=2.0 * T * ff * width)
        E, top, F = m["experts"], m["top"], m["expert_ff"]
        logits = f32(T, E + 1)
        ms = timed(lambda: ops.moe_route(logits, E, top, gate_col=E), flush=flush)
        record(f"moe_route {label}", ms, nbytes=T * ((E + 1) * 4 + top * 8 + 4))
        chosen, weight, gate = ops.moe_route(logits, E, top, gate_col=E)
        ms = timed(lambda: ops.moe_layout(chosen, E, torch.bfloat16, width, F), flush=flush)
        record(f"moe layout {label}", ms)
        lay = ops.moe_layout(chosen, E, torch.bfloat16, width, F)
        w_egu, w_ed = bf(E, 2 * F, width), bf(E, width, F)
        used = min(E, T * top)
        ms = timed(lambda: ops.moe_experts_up(xb, w_egu, lay, top), flush=flush)
        record(f"grouped gated product {label}", ms, nbytes=(used * 2 * F * width + T * width + T * top * F) * 2,
               flops=4.0 * T * top * F * width)
        act = ops.moe_experts_up(xb, w_egu, lay, top)
        ms = timed(lambda: ops.moe_experts_down(act, w_ed, lay), flush=flush)
        record(f"grouped down product {label}", ms, nbytes=(used * F * width + T * top * F) * 2 + T * top * width * 4,
               flops=2.0 * T * top * F * width)
        y = ops.moe_experts_down(act, w_ed, lay)
        shared = f32(T, width)
        ms = timed(lambda: ops.moe_combine(y, lay.pos_of, weight, shared, gate), flush=flush)
        record(f"moe_combine {label}", ms, nbytes=T * width * 4 * (top + 2))
        # ---- the sum that closes a sublayer: x += norm(product), and the norm that opens the next one
        x, a, w1 = f32(T, width), f32(T, width), bf(width)
        ms = timed(lambda: ops.stream_norm_add(x, a, w1, 1e-6, next_weight=w1), flush=flush)
        record(f"stream_norm_add + next norm {label}", ms, nbytes=T * width * (4 + 4 + 4 + 2))
        ms = timed(lambda: ops.stream_norm_add(x, a, w1, 1e-6, copy=True), flush=flush)
        record(f"ritizen stream_norm_add {label}", ms, nbytes=T * width * (4 + 4 + 4 + 2))
        xq, delta = bf(T, width), bf(T, width)
        ms = timed(lambda: ops.add_rmsnorm(xq, w1, 1e-6, delta=delta), flush=flush)
        record(f"qwen2 add + norm {label}", ms, nbytes=T * width * 8)
    ops.take_device_errors()
    return rows


def run_arch_bukatar(args):
    shape, layers = args.shape, args.layers or 4
    pk, pk_src = peaks()
    qcfg = dict(SHAPES[shape], num_hidden_layers=layers)
    folders = {"bukatar": arch_folder(bukatar_config(shape, layers), f"bukatar_{shape}_L{layers}"),
               "ritizen": arch_folder(ritizen_config(shape, layers), f"ritizen_{shape}_L{layers}"),
               "qwen2": model_folder(SHAPES[shape], layers)}
    clocks = ClockSampler()
    with clocks:
        models = {name: model_points(folder, args.batch, args.prompt_len, PREFILL_TOKENS, 20)
                  for name, folder in folders.items()}
        kernels = kernel_points_bukatar(shape, args.batch, args.prompt_len + 512, PREFILL_TOKENS, pk)
    print(json.dumps({
        "arch": "bukatar", "beside": ["ritizen", "qwen2"], "shape": shape, "layers": layers, "batch": args.batch,
        "prompt_len": args.prompt_len, "prefill_tokens": PREFILL_TOKENS, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02) seed 0", "bukatar_mixers": BUKATAR_SHAPES[shape],
        "hidden": qcfg["hidden_size"], "intermediate": qcfg["intermediate_size"], "vocab": qcfg["vocab_size"],
        "models": models, "kernels": kernels, "peaks": dict(pk, source=pk_src), "clocks": clocks.summary()}))
    return 0


# ----------------------------------------------------------------------------------------
# --arch kupedra: the Kupedra design beside Bukatar and Qwen2 at equal layer sizes (random weights)
# ----------------------------------------------------------------------------------------
KUPEDRA_SHAPES = {
    # width and vocabulary of the Qwen2.5 shape of the same name; attention heads as there; the matrix memory with
    # heads x vdim = width; experts as in the Bukatar shape of the same name (a token's share has the dense
    # feed-forward's rows); four streams
    "0.5B": dict(heads=14, kv_heads=2, dim=64, mem_heads=14, mem_dim=64, mem_vdim=64, experts=8, top=2, expert_ff=1536,
                 shared_ff=1792, streams=4, bias_rows=32, bias_max=1024.0),
    "1.5B": dict(heads=12, kv_heads=2, dim=128, mem_heads=12, mem_dim=128, mem_vdim=128, experts=8, top=2, expert_ff=2816,
                 shared_ff=3328, streams=4, bias_rows=32, bias_max=2048.0),
}


def kupedra_config(shape, layers):
    """Layers alternate: the side-by-side mixer (attention with a distance table beside a matrix memory), then the
    rotary attention; every layer with routed experts."""
    q, m = SHAPES[shape], KUPEDRA_SHAPES[shape]
    moe = {"kind": "moe", "router": {"experts": m["experts"], "top": m["top"]},
           "expert": {"ff": m["expert_ff"], "limit": 7.0}, "shared": {"ff": m["shared_ff"], "limit": 7.0}}
    D = m["dim"]
    att = {"heads": m["heads"], "kv_heads": m["kv_heads"], "dim": D, "vdim": D}
    kinds = [
        lambda: {"type": "parallel", "mlp": moe,
                 "mixer": {"left": dict(att, scale=D ** -0.5, bias_max=m["bias_max"], bias_rows=m["bias_rows"],
                                        q_temp={"coef": 0.1, "every": 256}),
                           "right": {"heads": m["mem_heads"], "dim": m["mem_dim"], "vdim": m["mem_vdim"], "gate_cap": 15.0}}},
        lambda: {"type": "attention", "mlp": moe,
                 "mixer": dict(att, scale=D ** -0.5, rot={"base": 10000.0, "dims": D // 2, "scaling": {"factor": 4.0}})},
    ]
    return {"architecture": "Kupedra", "vocab": q["vocab_size"], "width": q["hidden_size"], "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0}, "logit_scale": 1.0, "streams": m["streams"], "max_positions": 4096,
            "layers": [kinds[i % 2]() for i in range(layers)]}


def kernel_points_kupedra(shape, batch, ctx_len, prefill_tokens, pk):
    """The Kupedra design's own kernels beside the like kernels of Bukatar (the attention's store, the attention
    itself, the sum that closes a sublayer, the experts' products), of Ritizen (the recurrence with a decay per
    token) and of Qwen2 at the shape's sizes, each alone between CUDA events with L2 flushed: milliseconds and the
    fraction of the roofline (measured copy bandwidth for kernels that stream, measured bf16 product rate for the
    attention kernels and the products of a prompt)."""
    import torch
    from llm_inference_lab_b200.kernels import ops

    dev = torch.device("cuda:0")
    q, m, rz = SHAPES[shape], KUPEDRA_SHAPES[shape], RITIZEN_SHAPES[shape]
    width, ff = q["hidden_size"], q["intermediate_size"]
    flush = torch.zeros((160 << 20,), dtype=torch.int16, device=dev)
    bw, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    rows = {}

    def record(name, ms, nbytes=None, flops=None):
        entry = {"ms": round(ms, 4)}
        if nbytes is not None:
            entry.update(gbs=round(nbytes / (ms / 1e3) / 1e9, 1), frac_hbm=round(nbytes / (ms / 1e3) / bw, 4))
        if flops is not None:
            entry.update(tflops=round(flops / (ms / 1e3) / 1e12, 2), frac_bf16=round(flops / (ms / 1e3) / tf, 4))
        rows[name] = entry

    bf = lambda *s: (0.5 * torch.randn(*s, device=dev)).to(torch.bfloat16)  # noqa: E731
    f32 = lambda *s: 0.5 * torch.randn(*s, device=dev)  # noqa: E731
    S = m["streams"]
    for label, q_lens, pos0 in (("prefill", [prefill_tokens], [0]), ("decode", [1] * batch, [ctx_len] * batch)):
        T, B = sum(q_lens), len(q_lens)
        ctx, pages = bench_ctx(q_lens, pos0, PAGE_SIZE, dev)
        # ---- the residual of several streams: the write of all streams with the next sublayer's read and norm
        X, y, g1 = f32(T, S, width), f32(T, width), bf(1)
        c_in, c_out, mix = torch.rand(S, device=dev), torch.rand(S, device=dev), torch.rand(S, S, device=dev)
        ms = timed(lambda: ops.hyper_write(X, y, mix, c_out, c_in, g1, 1e-6), flush=flush)
        record(f"hyper_write + next read and norm {label}", ms, nbytes=T * width * (8 * S + 4 + 2))
        ms = timed(lambda: ops.hyper_read_norm(X, c_in, g1, 1e-6), flush=flush)
        record(f"hyper_read_norm {label}", ms, nbytes=T * width * (4 * S + 2))
        x, a, w1 = f32(T, width), f32(T, width), bf(width)
        ms = timed(lambda: ops.stream_norm_add(x, a, w1, 1e-6, next_weight=w1), flush=flush)
        record(f"bukatar stream_norm_add + next norm {label}", ms, nbytes=T * width * (4 + 4 + 4 + 2))
        b2 = f32(T, width)
        ms = timed(lambda: ops.normed_sum(a, w1, 0.5, b2, w1, 0.5, 1e-6), flush=flush)
        record(f"normed_sum {label}", ms, nbytes=T * width * 12)
        # ---- attention: rotation, norm per head, temperatures and the paged store; then the kernels with a
        # distance table and learned sinks, beside plain causal attention with the extra one over the same pages
        nq, nkv, D = m["heads"], m["kv_heads"], m["dim"]
        hd = ops.padded_head(D, D)
        ck, cv = bf(pages, nkv, PAGE_SIZE, hd), bf(pages, nkv, PAGE_SIZE, hd)
        aproj = f32(T, (nq + 2 * nkv) * D)
        inv, temps, wn = torch.rand(D // 4, device=dev), torch.rand(nq, device=dev), bf(D)
        slots = ctx.groups[0].row_slot
        ms = timed(lambda: ops.head_prep_store(aproj, None, ctx.row_pos, inv, D // 2, slots, ck, cv, nq, nkv, D, D, hd,
                                               nq * D, (nq + nkv) * D, torch.bfloat16, norm_eps=1e-6, q_head_scale=temps),
                   flush=flush)
        record(f"head_prep_store rotation + unit norm + temperature {label}", ms,
               nbytes=T * ((nq + 2 * nkv) * D * 4 + (nq + 2 * nkv) * hd * 2))
        ms = timed(lambda: ops.head_prep_store(aproj, None, ctx.row_pos, None, 0, slots, ck, cv, nq, nkv, D, D, hd, nq * D,
                                               (nq + nkv) * D, torch.bfloat16, norm_eps=1e-6, q_norm_w=wn, k_norm_w=wn,
                                               temp_coef=0.1, temp_every=256), flush=flush)
        record(f"head_prep_store weighted norm + position temperature {label}", ms,
               nbytes=T * ((nq + 2 * nkv) * D * 4 + (nq + 2 * nkv) * hd * 2))
        ab = bf((nq + nkv) * D)
        ms = timed(lambda: ops.rope_pairs_store(aproj, ab, ctx.row_pos, inv, D // 2, slots, ck, cv, nq, nkv, D, D, hd,
                                                nq * D, nq * D, torch.bfloat16), flush=flush)
        record(f"bukatar rope_pairs_store {label}", ms, nbytes=T * ((nq + nkv) * D * 4 + (nq + 2 * nkv) * hd * 2))
        qq = bf(T, nq * hd)
        table, sinks = f32(nq, int(m["bias_max"]) + 1), f32(nq)
        all_pairs = sum(sum(p + i + 1 for i in range(n)) for p, n in zip(pos0, q_lens))
        keys = sum(p + n for p, n in zip(pos0, q_lens))
        for name, kw in (("causal + one", dict(sink_one=True)), ("distance table + learned sink", dict(sink=sinks, dist_bias=table)),
                         ("learned sink", dict(sink=sinks))):
            ms = timed(lambda: ops.attention(qq, ck, cv, ctx, ctx.groups[0], nq, nkv, hd, 0, D ** -0.5, **kw), flush=flush)
            record(f"attention {name} {label}", ms, nbytes=keys * 2 * nkv * hd * 2 + 2 * T * nq * hd * 2,
                   flops=4.0 * all_pairs * nq * hd)
        # ---- the matrix memory: gates, the walk of the running maximum, the recurrence, the finish; beside
        # Ritizen's state-space walk (the same recurrence kernel with a decay per token)
        H, N, V = m["mem_heads"], m["mem_dim"], m["mem_vdim"]
        vpad = ops.memory_value_width(V)
        mproj = f32(T, 2 * H * N + 2 * H * V + 2 * H)
        b_i = bf(H)
        S_state, m_state = torch.zeros(B, H, N, vpad, device=dev), torch.zeros(B, H, device=dev)

        def memory():
            gates, values = ops.memory_gates(mproj, 2 * H * N, 2 * H * N + 2 * H * V, 2 * H * N + 2 * H * V + H, b_i, b_i, H, V, 15.0)
            mm = ops.memory_stabilize(gates, m_state, ctx)
            o = ops.decay_scan(mproj[:, : H * N], mproj[:, H * N: 2 * H * N], values, S_state, ctx, H, H, N, vpad,
                               a_tok=gates[:, 0, :], s_tok=gates[:, 1, :])
            return ops.memory_finish(o, mm, mproj[:, 2 * H * N + H * V: 2 * H * N + 2 * H * V], bf(H * V), ctx, H, V,
                                     N ** -0.5, 1e-6, 1e-6)

        ms = timed(memory, flush=flush)
        mem_bytes = T * (2 * H * N + 2 * H * V + 2 * H) * 4 + T * H * vpad * 8 + T * H * V * 2 + 2 * S_state.numel() * 4
        record(f"matrix memory (gates, maximum, recurrence, finish) {label}", ms, nbytes=mem_bytes,
               flops=None if label == "decode" else 4.0 * T * H * N * vpad)
        gates, values = ops.memory_gates(mproj, 2 * H * N, 2 * H * N + 2 * H * V, 2 * H * N + 2 * H * V + H, b_i, b_i, H, V, 15.0)
        ms = timed(lambda: ops.memory_stabilize(gates.clone(), m_state, ctx), flush=flush)
        record(f"memory_stabilize (with a copy of the gates) {label}", ms)
        ms = timed(lambda: ops.decay_scan(mproj[:, : H * N], mproj[:, H * N: 2 * H * N], values, S_state, ctx, H, H, N, vpad,
                                          a_tok=gates[:, 0, :], s_tok=gates[:, 1, :]), flush=flush)
        record(f"matrix memory, the recurrence alone {label}", ms,
               nbytes=T * (2 * H * N + 2 * H * vpad + 2 * H) * 4 + 2 * S_state.numel() * 4,
               flops=None if label == "decode" else 4.0 * T * H * N * vpad)
        H2, N2, V2, G2 = rz["ssm_heads"], rz["ssm_state"], rz["ssm_vdim"], rz["ssm_groups"]
        conv = f32(T, H2 * V2 + 2 * G2 * N2)
        a_tok, s_tok = torch.rand(T, H2, device=dev), torch.rand(T, H2, device=dev)
        state2 = torch.zeros(B, H2, N2, V2, device=dev)
        ms = timed(lambda: ops.decay_scan(conv[:, H2 * V2 + G2 * N2:], conv[:, H2 * V2: H2 * V2 + G2 * N2], conv[:, : H2 * V2],
                                          state2, ctx, H2, G2, N2, V2, a_tok=a_tok, s_tok=s_tok), flush=flush)
        record(f"ritizen decay_scan decay per token {label}", ms,
               nbytes=T * (2 * G2 * N2 + 2 * H2 * V2 + 2 * H2) * 4 + 2 * state2.numel() * 4,
               flops=None if label == "decode" else 4.0 * T * H2 * N2 * V2)
        # ---- the experts: the capped gate in the products' epilogues beside the SiLU gate
        xb = bf(T, width)
        w_gu = bf(2 * ff, width)
        for name, limit in (("capped", 7.0), ("qwen2 SiLU", 0.0)):
            ms = timed(lambda: ops.linear_gated(xb, w_gu, limit=limit), flush=flush)
            record(f"gated product, {name} gate {label}", ms, nbytes=(2 * ff * width + T * (width + ff)) * 2,
                   flops=4.0 * T * ff * width)
        E, top, F = m["experts"], m["top"], m["expert_ff"]
        logits = f32(T, E + 1)
        ms = timed(lambda: ops.moe_route(logits, E, top, gate_col=E, renorm=False), flush=flush)
        record(f"moe_route, scores as they are {label}", ms, nbytes=T * ((E + 1) * 4 + top * 8 + 4))
        chosen, weight, gate = ops.moe_route(logits, E, top, gate_col=E, renorm=False)
        lay = ops.moe_layout(chosen, E, torch.bfloat16, width, F)
        w_egu = bf(E, 2 * F, width)
        used = min(E, T * top)
        for name, limit in (("capped", 7.0), ("bukatar SiLU", 0.0)):
            ms = timed(lambda: ops.moe_experts_up(xb, w_egu, lay, top, limit=limit), flush=flush)
            record(f"grouped gated product, {name} gate {label}", ms,
                   nbytes=(used * 2 * F * width + T * width + T * top * F) * 2, flops=4.0 * T * top * F * width)
    ops.take_device_errors()
    return rows


def run_arch_kupedra(args):
    shape, layers = args.shape, args.layers or 4
    pk, pk_src = peaks()
    qcfg = dict(SHAPES[shape], num_hidden_layers=layers)
    folders = {"kupedra": arch_folder(kupedra_config(shape, layers), f"kupedra_{shape}_L{layers}"),
               "bukatar": arch_folder(bukatar_config(shape, layers), f"bukatar_{shape}_L{layers}"),
               "qwen2": model_folder(SHAPES[shape], layers)}
    clocks = ClockSampler()
    with clocks:
        models = {name: model_points(folder, args.batch, args.prompt_len, PREFILL_TOKENS, 20)
                  for name, folder in folders.items()}
        kernels = kernel_points_kupedra(shape, args.batch, args.prompt_len + 512, PREFILL_TOKENS, pk)
    print(json.dumps({
        "arch": "kupedra", "beside": ["bukatar", "qwen2"], "shape": shape, "layers": layers, "batch": args.batch,
        "prompt_len": args.prompt_len, "prefill_tokens": PREFILL_TOKENS, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02) seed 0", "kupedra_mixers": KUPEDRA_SHAPES[shape],
        "hidden": qcfg["hidden_size"], "intermediate": qcfg["intermediate_size"], "vocab": qcfg["vocab_size"],
        "models": models, "kernels": kernels, "peaks": dict(pk, source=pk_src), "clocks": clocks.summary()}))
    return 0


def kv_bytes_per_token(cfg, layers):
    d = cfg["hidden_size"] // cfg["num_attention_heads"]
    return 2 * layers * 2 * cfg["num_key_value_heads"] * d


def main() -> int:
    global PROMPT_LEN, PREFILL_TOKENS
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0,
                    help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--shape", default="0.5B", choices=sorted(SHAPES),
                    help="layer sizes of another model of the architecture (the headline is 0.5B)")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="tokens each request holds before decoding")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out decode at batch 1 and 64 and the prefill")
    ap.add_argument("--skip-e2e", action="store_true", help="leave out the run through LLM.generate")
    ap.add_argument("--no-graph", action="store_true",
                    help="time decode steps launched kernel by kernel instead of replayed from CUDA graphs")
    ap.add_argument("--serve", type=int, default=0, metavar="REQUESTS",
                    help="instead of the headline run: REQUESTS prompts of 128..2,048 tokens through LLM.generate "
                         "with 512 tokens a step and 128 new tokens each (continuous batching); prints its own line")
    ap.add_argument("--stack-stamps", action="store_true",
                    help="run a few eager decode steps with the decode stack's in-kernel clock on and print what "
                         "each kind of phase took")
    ap.add_argument("--arch", default="qwen2", choices=["qwen2", "sogulix", "ritizen", "bukatar", "kupedra"],
                    help="sogulix: instead of the headline run, prefill and decode throughput of the Sogulix design "
                         "beside Qwen2 at the layer sizes of --shape (0.5B or 1.5B; --layers, default 4), and each "
                         "of its kernels beside Qwen2's like kernel; prints its own line.  ritizen: the same for the "
                         "Ritizen design, beside Sogulix and Qwen2; bukatar: the same for the Bukatar design, beside "
                         "Ritizen and Qwen2; kupedra: the same for the Kupedra design, beside Bukatar and Qwen2")
    ap.add_argument("--only-prefill", type=int, default=0, metavar="TOKENS",
                    help="run only a prefill of TOKENS tokens a few times and print its time (for profiling)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "pochenai/llm-inference-lab is a Rust + cuTile engine: no cargo/rustc or cuTile toolchain "
                          "offline, and the offline pip install stops at metadata-generation-failed (its pyproject.toml holds no engine)"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": "this engine runs on one GPU; --gpus must be 1", "n_gpus": args.gpus}))
        return 2
    warmup = max(args.warmup, 3)
    steps = max(1, min(args.steps, NEW_TOKENS - warmup - 2))
    PROMPT_LEN = args.prompt_len
    cfg = SHAPES[args.shape]
    args.layers = args.layers or cfg["num_hidden_layers"]
    headline = args.shape == "0.5B" and PROMPT_LEN == 512
    max_seq = max(4096, PROMPT_LEN + NEW_TOKENS + PAGE_SIZE, args.only_prefill + PAGE_SIZE)
    live = max(64 if headline else 0, args.batch)      # requests that hold pages at the same time

    import numpy as np
    import torch
    from llm_inference_lab_b200.engine import Engine
    from llm_inference_lab_b200.engine.decode_graph import DecodeGraphs

    if args.arch == "sogulix":
        if args.shape not in SOGULIX_SHAPES:
            ap.error("--arch sogulix knows the shapes " + ", ".join(sorted(SOGULIX_SHAPES)))
        args.layers = 0 if args.layers == cfg["num_hidden_layers"] else args.layers
        return run_arch_sogulix(args)
    if args.arch == "ritizen":
        if args.shape not in RITIZEN_SHAPES:
            ap.error("--arch ritizen knows the shapes " + ", ".join(sorted(RITIZEN_SHAPES)))
        args.layers = 0 if args.layers == cfg["num_hidden_layers"] else args.layers
        return run_arch_ritizen(args)
    if args.arch == "bukatar":
        if args.shape not in BUKATAR_SHAPES:
            ap.error("--arch bukatar knows the shapes " + ", ".join(sorted(BUKATAR_SHAPES)))
        args.layers = 0 if args.layers == cfg["num_hidden_layers"] else args.layers
        return run_arch_bukatar(args)
    if args.arch == "kupedra":
        if args.shape not in KUPEDRA_SHAPES:
            ap.error("--arch kupedra knows the shapes " + ", ".join(sorted(KUPEDRA_SHAPES)))
        args.layers = 0 if args.layers == cfg["num_hidden_layers"] else args.layers
        return run_arch_kupedra(args)
    folder = model_folder(cfg, args.layers)
    pk, pk_src = peaks()
    if args.serve:
        clocks = ClockSampler()
        with clocks:
            out = run_serve(folder, cfg, args.layers, args.serve, 512, 128, max(max_seq, 2048 + 128 + PAGE_SIZE),
                            graph=not args.no_graph)
        out["decode_hbm_frac"] = round(out["decode_hbm_gbs"] / pk["hbm_gbs"], 4)
        out.update({"model": f"Qwen2.5-{args.shape} shape", "layers": args.layers,
                    "layers_of_config": cfg["num_hidden_layers"], "dtype": "bf16",
                    "mode": "eager launches" if args.no_graph else "cuda graphs", "peaks": pk_src,
                    "clocks": clocks.summary()})
        print(json.dumps(out))
        return 0
    rng = np.random.default_rng(0)
    engine = Engine(folder, "bf16", max_tokens=live * (PROMPT_LEN + NEW_TOKENS + PAGE_SIZE) + max(4096, args.only_prefill),
                    page_size=PAGE_SIZE,
                    max_requests=live, max_batch_tokens=max(8192, PROMPT_LEN, args.only_prefill), max_seq_len=max_seq)
    graphs = DecodeGraphs(engine)
    engine.enable_step_graphs()   # a prefill of a repeating shape is replayed from a CUDA graph

    if args.stack_stamps:
        print(json.dumps(run_stack_stamps(engine, args.batch, rng)))
        return 0
    if args.only_prefill:
        PREFILL_TOKENS = args.only_prefill
        pms = run_prefill(engine, rng, repeats=2)
        print(json.dumps({"prefill_tokens": PREFILL_TOKENS, "ms": round(pms, 4), "layers": args.layers,
                          "tokens_per_s": round(PREFILL_TOKENS / (pms / 1e3), 1)}))
        return 0

    # The timed region (K steps between two events) is taken R times in a row, as far as the requests'
    # budgets of new tokens allow; the line reports the median region, with the fastest and the slowest.
    repeats = max(1, min(5, (NEW_TOKENS - warmup - 2) // steps))
    clocks = ClockSampler()
    regions = run_decode(engine, None if args.no_graph else graphs, args.batch, steps, warmup, rng, clocks, repeats)
    ms, launches, mean_ctx = median_region(regions)
    value = args.batch * steps / (ms / 1e3)
    nbytes = decode_bytes(cfg, args.layers, args.batch, mean_ctx)
    achieved = nbytes / (ms / steps / 1e3) / 1e9

    line = {
        "metric": f"decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Qwen2.5-{args.shape})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms / steps, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02) seed 0, uniform-random token ids",
        "config": {
            "model": f"Qwen2.5-{args.shape} shape", "global_batch": args.batch, "seq_len": max_seq,
            "parallelism": "single-gpu",
            "layers": args.layers, "layers_of_config": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "rope_theta": cfg["rope_theta"], "tied_embeddings": cfg["tie_word_embeddings"],
            "prompt_len": PROMPT_LEN, "new_tokens": NEW_TOKENS, "page_size": PAGE_SIZE,
            "decode": ("eager launches" if args.no_graph else "cuda-graph") + ", device feedback",
            "l2": f"inputs larger than L2 ({nbytes / 1e9:.1f} GB of weights and cache per step)",
            "peaks": pk_src},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "gpu_launches": launches,
        "repeats": {"n": len(regions), "ms_per_step_min": round(min(r[0] for r in regions) / steps, 4),
                    "ms_per_step_max": round(max(r[0] for r in regions) / steps, 4)},
        "clocks": clocks.summary(),
    }
    if not args.skip_points:
        pms = run_prefill(engine, rng)
        flops = prefill_flops(cfg, args.layers, PREFILL_TOKENS)
        line["prefill"] = {"value": round(PREFILL_TOKENS / (pms / 1e3), 1), "tokens": PREFILL_TOKENS,
                           "ms": round(pms, 4), "frac": round(flops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
        points = {}
        for b in ((1, 64) if headline else ()):
            k = min(steps, 100)
            bms, _, _ = median_region(run_decode(engine, graphs, b, k, warmup, rng, repeats=min(repeats, 3)))
            points[f"decode_b{b}"] = round(b * k / (bms / 1e3), 1)
        if not args.no_graph:
            # the same steps launched kernel by kernel: the reference reports both modes
            k = min(steps, 100)
            ems, _, _ = median_region(run_decode(engine, None, args.batch, k, warmup, rng, repeats=min(repeats, 3)))
            points[f"decode_b{args.batch}_eager"] = round(args.batch * k / (ems / 1e3), 1)
        line["points"] = points
    del graphs, engine
    torch.cuda.empty_cache()
    if not args.skip_e2e and headline:
        try:
            line["e2e"] = {k: (round(v, 1) if isinstance(v, float) else v)
                           for k, v in run_e2e(folder, args.batch, steps, warmup).items()}
        except Exception as exc:  # noqa: BLE001 - the device-timed number stands on its own
            line["e2e"] = {"error": f"{type(exc).__name__}: {exc}"}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
