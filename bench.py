"""Serving benchmark: decode tokens per second of the Qwen1.5-MoE-A2.7B-sized model with
random weights (bfloat16) on one B200, plus prefill, roofline and end-to-end figures; in the same
line, the same measurements at the layer sizes of Qwen2-57B-A14B (`sizes_57b`) and a
continuous-batching workload on the windowed variant of the model (`serving`).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --no-extras             # the headline model only
    python bench.py --workload serving      # the continuous-batching workload alone, a line of its own
    python bench.py --sizes 57b             # the larger model alone as the headline
    python bench.py --workload sweep        # decode at 1k-32k tokens of context, prompts of 8k and 16k
    python bench.py --workload kernels      # the weight-streaming product alone, by shape and row length

A step is one decode step of the whole batch.  One JSON line is printed.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Layer sizes of the model the benchmark is quoted on (Qwen1.5-MoE-A2.7B).
MODEL = dict(
    architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe",
    num_hidden_layers=24, hidden_size=2048, num_attention_heads=16, num_key_value_heads=16, head_dim=128,
    num_experts=60, num_experts_per_tok=4, moe_intermediate_size=1408, shared_expert_intermediate_size=5632,
    norm_topk_prob=False, decoder_sparse_step=1, intermediate_size=5632, vocab_size=151936, rope_theta=1000000.0,
    rms_norm_eps=1e-6, use_sliding_window=False, tie_word_embeddings=False, max_position_embeddings=4096)
MODEL_A = dict(MODEL)
FULL_LAYERS = MODEL["num_hidden_layers"]
MODEL_NAME = "Qwen1.5-MoE-A2.7B"
# The larger model of the same family (--sizes 57b; about 114 GB of weights with all 28 layers).
SIZES_57B = dict(num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
                 num_experts=64, num_experts_per_tok=8, moe_intermediate_size=2560,
                 shared_expert_intermediate_size=20480, intermediate_size=20480)


def peaks():
    """Measured peaks if the driver wrote them, else this pool's earlier measurement."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p.get("bf16_tflops_sustained") or p["bf16_tflops"]),
                        source="measured")
        except (KeyError, ValueError, json.JSONDecodeError):
            pass
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0, t1):
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.samples:
            if not (t0 - 0.05 <= t <= t1 + 0.15):
                continue
            parts = [x.strip() for x in line.split(",")]
            try:
                mhz.append(int(float(parts[0])))
                mx = max(mx, int(float(parts[1])))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def weight_bytes_per_decode_step(cfg, batch, layers, esz=2, distinct=None):
    """Bytes a decode step has to read: every weight it uses once.  Routed experts: `distinct` experts
    with rows per layer (the mean over the layers of what the step's own routing gave); without it, the
    expected number of distinct experts a batch of `batch` tokens touches."""
    H, Q, KV = cfg.hidden_size, cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    E, k, I, Is = cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size
    attn = ((Q + 2 * KV) * H + H * Q) * esz
    if distinct is None:
        distinct = E * (1.0 - (1.0 - k / E) ** batch)
    moe = (E + 1) * H * esz + distinct * 3 * I * H * esz + 3 * Is * H * esz
    head = cfg.vocab_size * H * esz
    return layers * (attn + moe) + head


def prefill_flops(cfg, T, layers):
    H, Q, KV = cfg.hidden_size, cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    E, k, I, Is = cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size
    per_tok = 2 * H * (Q + 2 * KV) + 2 * Q * H + 2 * H * (E + 1) + k * 6 * H * I + 6 * H * Is
    attn = 4 * Q * T * (T + 1) / 2          # QK^T and PV over the causal half
    return layers * (per_tok * T + attn) + 2 * H * cfg.vocab_size


def run_reference():
    print(json.dumps({"impl": "reference", "unavailable":
                      "vedantnimbarte/dlm is a Rust crate (Cargo.toml, no setup.py/pyproject.toml): pip cannot "
                      "install it offline and no Rust toolchain is present"}))
    return 0


def run_serving(args) -> dict:
    """Continuous batching on the windowed variant of the model: 64 requests, prompt lengths uniform in
    [256, 16384], output lengths uniform in [64, 512], seeded uniform token ids; a request arrives every
    second step, so portions of prompts (2,048-token portions) run beside decoded tokens in the same step.
    Everything goes through the scheduler and the Python entry point; one JSON line."""
    import torch

    from dlm_b200.config import Qwen2MoeConfig
    from dlm_b200.engine import Engine

    raw = dict(MODEL_A)
    raw.update(num_hidden_layers=args.layers, use_sliding_window=True, sliding_window=4096,
               max_window_layers=min(21, max(args.layers - 3, 0)), max_position_embeddings=32768)
    cfg = Qwen2MoeConfig.from_dict(raw)
    torch.cuda.set_device(0)
    p_lo, p_hi = args.serving_prompts
    n_req, pool_tokens, max_context = args.serving_requests, 262144, max(p_hi, 4096) + 512 + 64
    eng = Engine.from_random(cfg, seed=0, dtype="bfloat16", page_size=64, max_tokens=pool_tokens,
                             max_requests=n_req, max_step_tokens=2048, max_context=max_context)
    gen = torch.Generator().manual_seed(4)
    plen = torch.randint(p_lo, p_hi + 1, (n_req,), generator=gen).tolist()
    olen = torch.randint(64, 513, (n_req,), generator=gen).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for n in plen]
    # warm-up: one short request end to end (kernels loaded, graphs of its shapes captured)
    eng.generate([prompts[0][:300]], max_new_tokens=4)
    torch.cuda.synchronize()
    sampler = ClockSampler()
    sampler.start()
    t0 = time.time()
    submitted, produced, steps = 0, 0, 0
    # per step: time between two events around it, wall time, and whether it carried prompt tokens (the events
    # enclose the host's work inside the step too; what the host costs is in the scheduler's counters below)
    records, prompt_seen = [], eng.scheduler.stats().prompt_tokens
    while submitted < n_req or eng.scheduler.has_work():
        if submitted < n_req and steps % 2 == 0:
            eng.submit(prompts[submitted], max_new_tokens=olen[submitted])
            submitted += 1
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.perf_counter()
        e0.record()
        out = eng.run_step()
        e1.record()
        e1.synchronize()
        w1 = time.perf_counter()
        now = eng.scheduler.stats().prompt_tokens
        records.append((e0, e1, w1 - w0, now - prompt_seen, len(out)))
        prompt_seen = now
        produced += len(out)
        steps += 1
    torch.cuda.synchronize()
    t1 = time.time()
    kinds = {"decode_only": [], "with_prompt_le_256": [], "with_prompt_gt_256": []}
    for e0, e1, wall, ptoks, rows in records:
        kind = "decode_only" if ptoks == 0 else ("with_prompt_le_256" if ptoks <= 256 else "with_prompt_gt_256")
        kinds[kind].append((e0.elapsed_time(e1), 1e3 * wall))
    step_kinds = {k: {"steps": len(v), "device_ms_mean": round(sum(a for a, _ in v) / len(v), 3),
                      "wall_ms_mean": round(sum(b for _, b in v) / len(v), 3)} for k, v in kinds.items() if v}
    time.sleep(0.2)
    sampler.stop()
    clocks = sampler.summary(t0, t1)
    st = eng.stats()
    ok = st["finished"] >= n_req and produced == sum(olen)
    line = {
        "metric": f"serving: generated tok/s, {n_req} requests, prompts {p_lo}-{p_hi}, outputs 64-512, continuous batching "
                  "(Qwen1.5-MoE-A2.7B sizes, layers 21-23 windowed at 4096, bf16, random weights)",
        "value": round(produced / (t1 - t0), 2), "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True,
        "dtype": "bf16", "data": "synthetic: seeded uniform token ids, random weights N(0, 0.02)", "impl": "ours",
        "seconds": round(t1 - t0, 3), "generated_tokens": produced, "prompt_tokens": sum(plen),
        "prompt_tok_s": round(sum(plen) / (t1 - t0), 1), "steps": steps, "complete": ok,
        "config": {"model": "Qwen1.5-MoE-A2.7B sizes, window", "requests": n_req, "layers": args.layers,
                   "layers_full": MODEL_A["num_hidden_layers"], "pool_tokens": pool_tokens, "portion": 2048, "page_size": 64,
                   "arrivals": "one request every second step"},
        "scheduler": {k: st[k] for k in ("steps", "prompt_tokens", "decode_tokens", "preemptions", "finished",
                                         "graphs_recorded", "graph_record_seconds", "eager_steps",
                                         "eager_launch_seconds")},
        "pages": st["pages"], "clocks": clocks,
        # the steps by kind; the host's share: seconds spent recording decode graphs (the device idles) and
        # launching the steps that are not replayed (the device works meanwhile)
        "step_kinds": step_kinds,
        "host": {"graphs_recorded": st["graphs_recorded"], "graph_record_s": st["graph_record_seconds"],
                 "eager_steps": st["eager_steps"], "eager_launch_s": st["eager_launch_seconds"]},
    }
    del eng
    return line


class Measurement:
    """One model on the device and the measurements taken on it: decode steps at several batch sizes
    (device time of the replayed step, and end to end through run_step) and one 2,048-token prefill."""

    def __init__(self, raw, layers, prompt_len, context, max_batch, pk, page=64):
        import torch

        from dlm_b200.config import Qwen2MoeConfig
        from dlm_b200.engine import Engine
        self.torch = torch
        raw = dict(raw)
        raw["num_hidden_layers"] = layers
        self.cfg = Qwen2MoeConfig.from_dict(raw)
        self.layers, self.prompt_len, self.pk = layers, prompt_len, pk
        torch.cuda.set_device(0)
        self.page = page
        pool_tokens = max_batch * (prompt_len + 256) + 4096
        t_load = time.time()
        self.eng = Engine.from_random(self.cfg, seed=0, dtype="bfloat16", page_size=self.page, max_tokens=pool_tokens,
                                      max_requests=max_batch, max_step_tokens=2048, max_context=context)
        torch.cuda.synchronize()
        self.load_s = time.time() - t_load
        self.gen = torch.Generator().manual_seed(0)
        # the routing of every captured step: the permutation's offsets stay in the graph's memory
        self.offsets = []
        ops = self.eng.rt.ops
        route = ops.route

        def recording_route(*a, **kw):
            out = route(*a, **kw)
            self.offsets.append(out[3])          # (ids, wts, gate, offsets, rows, dest)
            return out
        ops.route = recording_route

    def close(self):
        import gc
        self.eng._graphs.clear()
        self.eng = None
        self.offsets = []
        gc.collect()
        self.torch.cuda.empty_cache()

    def prompts(self, n, length):
        return [self.torch.randint(0, self.cfg.vocab_size, (length,), generator=self.gen).tolist() for _ in range(n)]

    def decode(self, batch, steps, warmup, sample_clocks=False):
        """Prefills `batch` prompts through the scheduler, then times `steps` decode steps of the step
        function (device time) and the same number through run_step (end to end)."""
        torch, eng = self.torch, self.eng
        ids = [eng.submit(p, max_new_tokens=10 ** 6) for p in self.prompts(batch, self.prompt_len)]
        started = set()
        while len(started) < batch:                   # admit and prefill everything
            started.update(rid for rid, _ in eng.run_step())
        # every request now decodes one token per step
        self.offsets = []
        for _ in range(max(warmup, 3)):
            eng.run_step()
        torch.cuda.synchronize()
        # device time of the decode step itself: `steps` replays of the captured step (the step function
        # and the arg-max over its logits, all kernels of one decode step), no host work in between
        key = next(k for k in eng._graphs if k[0] == batch and k[1] >= self.prompt_len)
        ent = eng._graphs[key]
        sampler = ClockSampler()
        if sample_clocks:
            sampler.start()
            time.sleep(0.3)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.time()
        e0.record()
        for _ in range(steps):
            ent["graph"].replay()
        e1.record()
        torch.cuda.synchronize()
        t1 = time.time()
        dev_ms = e0.elapsed_time(e1)
        clocks = None
        if sample_clocks:
            time.sleep(0.2)
            sampler.stop()
            clocks = sampler.summary(t0, t1)
        # the experts that had rows in the replayed step, per layer (the last capture's offsets)
        distinct = None
        sparse = sum(1 for i in range(self.layers) if self.cfg.layer_is_sparse(i))
        if sparse and len(self.offsets) >= sparse:
            offs = torch.stack(self.offsets[-sparse:]).cpu()
            distinct = float(((offs[:, 1:] - offs[:, :-1]) > 0).sum(dim=1).double().mean())
        # end to end: wall clock around the public loop, host tokens in and out every step
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        produced = 0
        for _ in range(steps):
            produced += len(eng.run_step())
        torch.cuda.synchronize()
        w1 = time.perf_counter()
        ctx = eng.cache.manager.length(0) if eng.cache.manager.is_open(0) else self.prompt_len
        for i in ids:
            eng.abort(i)
        eng.scheduler.drain_finished()
        ms = dev_ms / steps
        kv_bytes = batch * (self.prompt_len + max(warmup, 3) + 2 + steps // 2) * eng.cache.bytes_per_token()
        step_bytes = weight_bytes_per_decode_step(self.cfg, batch, self.layers, distinct=distinct) + kv_bytes
        achieved = step_bytes / (ms / 1e3) / 1e9
        return dict(ms=ms, tok_s=batch * steps / (dev_ms / 1e3), e2e_tok_s=produced / (w1 - w0),
                    launches=ent["launches"] * steps, clocks=clocks, ctx=ctx, distinct=distinct,
                    step_bytes=step_bytes, achieved=achieved, frac=achieved / self.pk["hbm_gbs"],
                    h2d=int(eng.cache.last_h2d_bytes))

    def decode_sampled(self, batch, steps, temperature=0.8):
        """Tokens a second end to end through run_step with seeded temperature sampling (the sampling kernel
        and its host side on top of the replayed step)."""
        from dlm_b200.sampling import SamplingParams
        torch, eng = self.torch, self.eng
        ids = [eng.submit(p, SamplingParams(temperature=temperature, seed=i), max_new_tokens=10 ** 6)
               for i, p in enumerate(self.prompts(batch, self.prompt_len))]
        started = set()
        while len(started) < batch:
            started.update(rid for rid, _ in eng.run_step())
        for _ in range(3):
            eng.run_step()
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        produced = 0
        for _ in range(steps):
            produced += len(eng.run_step())
        torch.cuda.synchronize()
        w1 = time.perf_counter()
        for i in ids:
            eng.abort(i)
        eng.scheduler.drain_finished()
        return produced / (w1 - w0)

    def prefill(self, T=2048, repeats=4):
        torch, eng = self.torch, self.eng
        times = []
        for _ in range(repeats):
            s = eng.cache.open()
            toks = self.prompts(1, T)[0]
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.step([(s, toks, [T - 1])])
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
            eng.cache.close(s)
        pms = min(times[1:]) if len(times) > 1 else times[0]
        flops = prefill_flops(self.cfg, T, self.layers)
        return {"value": round(T / (pms / 1e3), 1), "tokens": T, "ms": round(pms, 3),
                "frac": round(flops / (pms / 1e3) / (self.pk["bf16_tflops"] * 1e12), 4),
                "peak_tflops": self.pk["bf16_tflops"], "all_ms": [round(t, 3) for t in times]}


def run_sweep(args, pk) -> dict:
    """Further contexts: decode steps at batch 1 / 8 / 64 with 1k to 32k tokens of context each (as far as the
    pool holds them), and prompts of 8k and 16k tokens prefilled in portions of 2,048, each with its fraction of
    the measured peak."""
    out = {"metric": "sweep over contexts (%s sizes, bf16, random weights)" % MODEL_NAME, "layers": args.layers,
           "layers_full": FULL_LAYERS, "decode": {}, "prefill": {}}
    for ctx in (1024, 4096, 8192, 16384, 32768):
        for b in (1, 8, 64):
            if b * ctx > 600_000:          # 64 x 16k and 64 x 32k would not fit beside the weights
                continue
            m = Measurement(MODEL, args.layers, ctx, ctx + 512, b, pk)
            r = m.decode(b, 8, 3)
            out["decode"][f"b{b}_ctx{ctx}"] = {"tok_s": round(r["tok_s"], 1), "ms": round(r["ms"], 3),
                                                "frac": round(r["frac"], 4)}
            m.close()
    import torch
    for plen in (8192, 16384):
        m = Measurement(MODEL, args.layers, plen, plen + 512, 1, pk)
        eng, times = m.eng, []
        for _ in range(2):
            s = eng.cache.open()
            toks = m.prompts(1, plen)[0]
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(0, plen, 2048):
                eng.step([(s, toks[i:i + 2048], [2047] if i + 2048 >= plen else [])])
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
            eng.cache.close(s)
        ms = min(times)
        flops = prefill_flops(m.cfg, plen, args.layers)
        out["prefill"][f"prompt{plen}"] = {"tok_s": round(plen / (ms / 1e3), 1), "ms": round(ms, 2),
                                           "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
        m.eng.rt.ops.check_errors()
        m.close()
    return out


def run_kernels(pk) -> dict:
    """The decode step's products alone, timed with CUDA events inside a captured graph, the weights rotated
    over several copies so that L2 does not hold them: the dense shapes (8 rows, the weight-streaming kernel), the
    routed experts' products at 1 / 8 / 64 tokens (whichever kernel the rule chooses: the weight-streaming one at
    1 and 8, the tcgen05 one at 64), and 8 rows against 256 MB of weights with rows of 512 to 4,096 elements."""
    import torch

    from dlm_b200.ops import native_ops
    ops = native_ops(fast=True)
    dev = "cuda"
    bf = torch.bfloat16

    def timed(fn, copies, reps=3):
        for c in range(copies):
            fn(c)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                for c in range(copies):
                    fn(c)
        g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(5):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1000 / (5 * reps * copies)

    out = {"metric": "the decode step's products alone: us and TB/s", "peak_gbs": pk["hbm_gbs"], "dense": {},
           "grouped": {}, "row_length": {}}
    for (N, K, kind) in [(6144, 2048, "store"), (2048, 2048, "add"), (11264, 2048, "swiglu"), (2048, 5632, "store"),
                         (151936, 2048, "store")]:
        copies = max(2, min(12, int(300e6 // (N * K * 2)) + 1))
        ws = [torch.randn(N, K, device=dev).to(bf) * 0.05 for _ in range(copies)]
        a = torch.randn(8, K, device=dev).to(bf)
        resid = torch.zeros(8, N, device=dev)
        fn = {"store": lambda c: ops.linear(a, ws[c], None, torch.float32),
              "add": lambda c: ops.linear_add(a, ws[c], resid),
              "swiglu": lambda c: ops.linear_swiglu(a, ws[c])}[kind]
        us = timed(fn, copies)
        out["dense"][f"{N}x{K}_{kind}"] = {"us": round(us, 2), "tb_s": round(N * K * 2 / us / 1e6, 2)}
        del ws
    E, k, H, I = MODEL_A["num_experts"], MODEL_A["num_experts_per_tok"], MODEL_A["hidden_size"], MODEL_A["moe_intermediate_size"]
    for T in (1, 8, 64):
        g = torch.Generator().manual_seed(T)
        ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).cuda()
        offsets, rows, _ = ops.moe_permute(ids, E)
        active = int(((offsets[1:] - offsets[:-1]) > 0).sum())
        wgu = [torch.randn(E, 2 * I, H, device=dev).to(bf) * 0.05 for _ in range(3)]
        wd = [torch.randn(E, H, I, device=dev).to(bf) * 0.05 for _ in range(3)]
        h = torch.randn(T, H, device=dev).to(bf)
        act = ops.grouped_swiglu(h, wgu[0], offsets, rows)
        u1 = timed(lambda c: ops.grouped_swiglu(h, wgu[c], offsets, rows), 3)
        u2 = timed(lambda c: ops.grouped_linear(act, wd[c], offsets), 3)
        out["grouped"][f"tokens{T}"] = {"experts_with_rows": active,
                                        "gate_up_us": round(u1, 2), "gate_up_tb_s": round(active * 2 * I * H * 2 / u1 / 1e6, 2),
                                        "down_us": round(u2, 2), "down_tb_s": round(active * I * H * 2 / u2 / 1e6, 2)}
        del wgu, wd
    for K in (512, 1024, 1408, 1536, 2048, 2816, 4096):
        N = (256 * 1024 * 1024 // 2) // K // 16 * 16
        ws = [torch.randn(N, K, device=dev).to(bf) for _ in range(2)]
        a = torch.randn(8, K, device=dev).to(bf)
        us = timed(lambda c: ops.linear(a, ws[c], None, torch.float32), 2)
        out["row_length"][f"K{K}"] = {"us": round(us, 1), "tb_s": round(N * K * 2 / us / 1e6, 2)}
        del ws
    ops.check_errors()
    return out


def layers_that_fit(raw, want, reserve_gb=40.0):
    """As many layers of `raw` (at most `want`) as the free device memory holds beside `reserve_gb` for
    the cache pool, the head, graphs and activations."""
    import torch
    H, I, Is, E = raw["hidden_size"], raw["moe_intermediate_size"], raw["shared_expert_intermediate_size"], raw["num_experts"]
    Q = raw["num_attention_heads"] * raw["head_dim"]
    KV = raw["num_key_value_heads"] * raw["head_dim"]
    per_layer = 2 * ((Q + 2 * KV) * H + H * Q + (E + 1) * H + E * 3 * I * H + 3 * Is * H)
    free, _ = torch.cuda.mem_get_info(0)
    fit = int((free - reserve_gb * 1e9) // per_layer)
    return max(1, min(want, fit))


def measure_57b(args, pk) -> dict:
    """The layer sizes of Qwen2-57B-A14B: decode at batch 1 / 8 / 64 (context 2,048) and a 2,048-token
    prefill, each with its fraction of the measured peak."""
    raw = dict(MODEL_A)
    raw.update(SIZES_57B)
    raw["max_position_embeddings"] = 4096
    full = SIZES_57B["num_hidden_layers"]
    layers = layers_that_fit(raw, full if args.layers_57b is None else args.layers_57b)
    m = Measurement(raw, layers, 2048, 4096, 64, pk)
    out = {"model": "Qwen2-57B-A14B sizes", "layers": layers, "layers_full": full, "prompt_len": 2048,
           "load_s": round(m.load_s, 1)}
    for b in (8, 1, 64):
        r = m.decode(b, max(4, args.steps // 4), 3, sample_clocks=(b == 8))
        out[f"decode_b{b}"] = round(r["tok_s"], 2)
        out[f"decode_b{b}_ms"] = round(r["ms"], 4)
        out[f"decode_b{b}_frac"] = round(r["frac"], 4)
        out[f"decode_b{b}_experts"] = r["distinct"]
        if b == 8:
            out["clocks"] = r["clocks"]
    out["prefill"] = m.prefill(2048, repeats=3)
    m.eng.rt.ops.check_errors()
    m.close()
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--page-size", type=int, default=64, help="tokens per page of the cache (16, 32, 64, 128, ...)")
    ap.add_argument("--serving-prompts", type=int, nargs=2, default=[256, 16384], metavar=("MIN", "MAX"),
                    help="prompt lengths of the serving workload (uniform in MIN..MAX)")
    ap.add_argument("--serving-requests", type=int, default=64, help="requests of the serving workload")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (reported)")
    ap.add_argument("--layers-57b", type=int, default=None, help="layers of the larger model in `sizes_57b` (default: all "
                    "28 if they fit)")
    ap.add_argument("--sizes", default="a2.7b", choices=["a2.7b", "57b"],
                    help="57b: the layer sizes of Qwen2-57B-A14B as the headline (no extras)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 and prefill measurements")
    ap.add_argument("--no-extras", action="store_true", help="skip `sizes_57b` and `serving`")
    ap.add_argument("--only-prefill", action="store_true", help="measure the 2,048-token prefill alone (for profiles)")
    ap.add_argument("--workload", default="decode", choices=["decode", "serving", "sweep", "kernels"],
                    help="serving: the continuous-batching workload on the windowed model, instead of the default line; "
                         "sweep: decode at contexts of 1k to 32k and prefill of longer prompts, a line of its own; "
                         "kernels: the weight-streaming product alone")
    args = ap.parse_args()
    global FULL_LAYERS, MODEL_NAME
    if args.sizes == "57b":
        MODEL.update(SIZES_57B)
        FULL_LAYERS, MODEL_NAME = SIZES_57B["num_hidden_layers"], "Qwen2-57B-A14B"
        args.no_extras = True
    if args.impl == "reference":
        return run_reference()
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.workload == "serving":
        if args.layers is None:
            args.layers = MODEL_A["num_hidden_layers"]
        line = run_serving(args)
        print(json.dumps(line))
        return 0 if line["complete"] else 1
    if args.layers is None:
        args.layers = FULL_LAYERS
    args.warmup = max(args.warmup, 3)
    pk = peaks()
    if args.workload == "sweep":
        print(json.dumps(run_sweep(args, pk)))
        return 0
    if args.workload == "kernels":
        print(json.dumps(run_kernels(pk)))
        return 0
    max_batch = 64 if not args.no_points else args.batch
    m = Measurement(MODEL, args.layers, args.prompt_len, args.context, max_batch, pk, page=args.page_size)
    cfg = m.cfg
    if args.only_prefill:
        pre = m.prefill(2048, repeats=3)
        print(json.dumps({"prefill_ms": pre["all_ms"], "tokens": 2048, "layers": args.layers}))
        return 0
    main_run = m.decode(args.batch, args.steps, args.warmup, sample_clocks=True)
    out = {
        "metric": "decode tok/s @ batch %d (%s sizes, bf16, random weights)" % (args.batch, MODEL_NAME),
        "value": round(main_run["tok_s"], 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform token ids, random weights N(0, 0.02)", "impl": "ours",
        "config": {
            "model": MODEL_NAME + " sizes", "global_batch": args.batch, "seq_len": args.context,
            "parallelism": "1 GPU", "prompt_len": args.prompt_len, "layers": args.layers, "layers_full": FULL_LAYERS,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "experts": cfg.num_experts, "top_k": cfg.num_experts_per_tok,
            "moe_inter": cfg.moe_intermediate_size, "shared_inter": cfg.shared_expert_intermediate_size,
            "vocab": cfg.vocab_size, "page_size": m.page,
            "l2": "inputs larger than L2: a step reads %.1f GB" % (main_run["step_bytes"] / 1e9),
            "timed": "K replays of the captured decode step (CUDA graph), CUDA events",
            "peaks": pk["source"]},
        "e2e": {"value": round(main_run["e2e_tok_s"], 2), "unit": "tokens/s",
                "h2d_bytes_per_step": main_run["h2d"], "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": int(main_run["launches"]),
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": round(main_run["achieved"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(main_run["frac"], 4), "experts_with_rows": main_run["distinct"]},
        "load_s": round(m.load_s, 1),
    }
    if not args.no_points:
        pts, fracs, e2e = {}, {f"decode_b{args.batch}": round(main_run["frac"], 4)}, {}
        for b in (1, 64):
            r = m.decode(b, max(8, args.steps // 2), 3)
            pts[f"decode_b{b}"] = round(r["tok_s"], 2)
            fracs[f"decode_b{b}"] = round(r["frac"], 4)
            e2e[f"decode_b{b}"] = round(r["e2e_tok_s"], 2)
        out["points"] = pts
        out["points_frac"] = fracs          # of the HBM peak, bytes from the experts each step really used
        out["points_e2e"] = e2e             # the same points through run_step, host tokens in and out
        out["e2e_sampled"] = {"value": round(m.decode_sampled(args.batch, args.steps), 2), "unit": "tokens/s",
                              "temperature": 0.8, "batch": args.batch}
        out["prefill"] = m.prefill(2048, repeats=4)
        out["prefill"].pop("all_ms")
    m.eng.rt.ops.check_errors()
    m.close()
    if not args.no_extras and not args.no_points:
        sv_args = argparse.Namespace(layers=MODEL_A["num_hidden_layers"])
        sv = run_serving(sv_args)
        out["serving"] = {"generated_tok_s": sv["value"], "prompt_tok_s": sv["prompt_tok_s"], "seconds": sv["seconds"],
                          "steps": sv["steps"], "mean_step_ms": round(1e3 * sv["seconds"] / max(sv["steps"], 1), 3),
                          "requests": sv["config"]["requests"], "layers": sv["config"]["layers"],
                          "prompt_tokens": sv["prompt_tokens"], "generated_tokens": sv["generated_tokens"],
                          "preemptions": sv["scheduler"]["preemptions"],
                          "high_water_pages": [p["high_water"] for p in sv["pages"]],
                          "pool_pages": [p["total"] for p in sv["pages"]], "complete": sv["complete"],
                          "host": sv["host"], "step_kinds": sv["step_kinds"],
                          "clocks": sv["clocks"]}
        import gc

        import torch
        gc.collect()
        torch.cuda.empty_cache()
        out["sizes_57b"] = measure_57b(args, pk)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
