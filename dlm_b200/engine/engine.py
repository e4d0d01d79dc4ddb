"""The engine: a model, its cache, one step function, a scheduler and a sampler.

``Engine.from_pretrained(dir)`` mirrors the reference's ``load_generator``
(src/loader.rs:340-346) and ``Engine.generate(prompt, ...)`` its
``Generator::generate(prompt, GenerationConfig)`` (src/generate.rs:338-373):
same option names, same defaults (16 new tokens, greedy, no end-of-sequence
token), the end-of-sequence token is part of the output.  Unlike the reference,
several prompts are run together: prompts are cut into portions under a token
budget and decoded tokens of other requests share the step.
"""
from __future__ import annotations

import time
from collections import OrderedDict
from typing import Iterable, Sequence

import torch

from ..build import load_host
from ..cache import ModelCache
from ..parts.base import Runtime
from ..sampling import RequestSampler, SamplingParams, sample_rows
from ..weights import load_model, random_model

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def _dtype(d) -> torch.dtype:
    if d not in _DTYPES:
        raise ValueError(f"dtype must be bfloat16 or float32, got {d!r}")
    return _DTYPES[d]


def make_runtime(dtype="bfloat16", device="cuda:0", ops=None) -> Runtime:
    """Runtime with the native kernels (the only product backend).  In 32-bit mode every
    product and the attention run on the FMA units."""
    dt = _dtype(dtype)
    if ops is None:
        from ..ops import native_ops
        torch.cuda.set_device(torch.device(device))
        ops = native_ops(fast=(dt == torch.bfloat16))
    return Runtime(device, dt, ops)


def _row_bucket(rows: int, cap: int) -> int:
    """The smallest of 1, 2, 3, 4, 6, 8, 12, 16, 24, 32, ... (powers of two and their one-and-a-half) that is
    at least ``rows``, but no more than ``cap`` (and never less than ``rows``)."""
    p = 1
    while True:
        for b in (p, p + p // 2):
            if b >= rows:
                return max(rows, min(b, cap))
        p *= 2


class Engine:
    def __init__(self, config, model, *, page_size: int = 64, num_pages: int | None = None,
                 max_tokens: int | None = None, max_requests: int = 64, max_step_tokens: int = 2048,
                 max_context: int | None = None):
        self.config, self.model, self.rt = config, model, model.rt
        if max_context is None:
            max_context = getattr(config, "max_position_embeddings", None) or 4096
        self.max_context = int(max_context)
        if num_pages is None and max_tokens is None:
            max_tokens = min(self.max_context * max_requests, self._tokens_that_fit(page_size))
        self.cache = ModelCache(model, page_size=page_size, num_pages=num_pages, max_tokens=max_tokens,
                                num_slots=max_requests)
        host = load_host()
        self.scheduler = host.Scheduler(self.cache.manager, host.SchedulerConfig(
            max_step_tokens=int(max_step_tokens), max_step_requests=int(max_requests),
            max_context=self.max_context, vocab_size=int(model.spec.vocab_size)))
        # replayed CUDA graphs of pure decode steps, keyed by (rows, bucket of the longest request); at most
        # `max_graphs` are kept, the least recently used goes first.  Not for a model with a part that
        # synchronises with the host inside its forward.
        self.use_graphs = (self.rt.device.type == "cuda" and hasattr(self.rt.ops, "launches")
                           and all(part.graph_safe for part in self._all_parts()))
        self.max_graphs = 32
        self._graphs: "OrderedDict[tuple[int, int], dict]" = OrderedDict()
        self.graphs_recorded = 0          # how many decode graphs were recorded so far
        self.graph_record_seconds = 0.0   # host time spent recording them
        self.eager_steps = 0              # steps launched kernel by kernel (not replayed)
        self.eager_launch_seconds = 0.0   # host time spent launching them (the device works meanwhile)
        self._graph_pool = None
        self._samplers: dict[int, RequestSampler] = {}
        self._results: dict[int, list[int]] = {}
        self._reasons: dict[int, str] = {}
        self._next_id = 0
        self.last_logits: torch.Tensor | None = None

    # ------------------------------------------------------------ builders
    @classmethod
    def from_pretrained(cls, path: str, dtype="bfloat16", device="cuda:0", ops=None, **kw) -> "Engine":
        rt = make_runtime(dtype, device, ops)
        cfg, model = load_model(path, rt)
        return cls(cfg, model, **kw)

    @classmethod
    def from_random(cls, config, seed: int = 0, dtype="bfloat16", device="cuda:0", ops=None, **kw) -> "Engine":
        rt = make_runtime(dtype, device, ops)
        cfg, model = random_model(config, seed, rt)
        return cls(cfg, model, **kw)

    def _all_parts(self):
        for block in self.model.blocks:
            yield block
            for _, part in block.children():
                yield part

    def _tokens_that_fit(self, page_size: int) -> int:
        per_token = 0
        for ci, (need, _, owner) in enumerate(self.model.cache_needs()):
            if need is not None and owner == ci:
                per_token += need.elements_per_token() * (2 if self.rt.dtype == torch.bfloat16 else 4)
        per_token = max(per_token, 1)
        if self.rt.device.type == "cuda":
            free, _ = torch.cuda.mem_get_info(self.rt.device)
            budget = int(free * 0.6)
        else:
            budget = 1 << 28
        return max(page_size, budget // per_token)

    # ---------------------------------------------------------- step function
    def step(self, items: Sequence[tuple[int, Sequence[int], Sequence[int]]]) -> torch.Tensor:
        """Runs one batch.  ``items``: ``(slot, next tokens, wanted places)`` for each request
        of the step; slots come from ``cache.open()``.  Takes the pages the tokens need,
        runs only these tokens against the cache and returns the logits at the wanted
        places, ``[wanted, vocab]`` in 32-bit, in the order of the items."""
        self.cache.append([(s, len(t)) for s, t, _ in items])
        return self._run(items)

    def _run(self, items) -> torch.Tensor:
        t0 = time.perf_counter()
        batch = self.cache.make_batch(items)
        out = self.model.step(batch, self.cache)
        self.eager_steps += 1
        self.eager_launch_seconds += time.perf_counter() - t0
        return out

    # ------------------------------------------------- replayed decode steps
    def _run_decode(self, items):
        """A pure decode step through its graph.  Returns (logits, greedy tokens) on the device and, from a
        replayed graph, the greedy tokens in pinned host memory (valid once the stream has been waited for).

        A graph is the step function and the arg-max over its logits for `rows` requests none of which
        holds more than `bucket` tokens; everything its kernels read that changes from step to step lies
        in one device buffer of fixed layout, refilled before every replay.  The first step of a new
        (rows, bucket) runs eagerly on that buffer (first-call set-up of the kernels must not fall into a
        capture) and its result is the step's result; the graph is then recorded for the steps after it.
        Recording runs nothing, so every step runs exactly once, which per-request state needs."""
        cache, ops = self.cache, self.rt.ops
        slots = [int(s) for s, _, _ in items]
        longest = cache.manager.max_length(slots)
        bucket = 256
        while bucket < longest:
            bucket *= 2
        bucket = min(bucket, max(self.max_context, longest))
        # rows are padded up to the next of 1, 2, 3, 4, 6, 8, 12, 16, 24, ... (at most half more), so that a batch
        # that shrinks request by request does not ask for a new graph at every size
        rows = len(items)
        padded = _row_bucket(rows, self.cache.num_slots)
        key = (padded, bucket)
        ent = self._graphs.get(key)
        if ent is not None:
            # the graph copies the metadata from its pinned buffer itself and leaves the tokens in another; the
            # step before this one has been waited for (its tokens were read), so the buffers are free
            self._graphs.move_to_end(key)
            stage = ent["stage"]
            cache.manager.pack_decode(slots, [int(t[0]) for _, t, _ in items], ent["layout"], stage.data_ptr(),
                                      stage.numel())
            cache.last_h2d_bytes = 4 * ent["layout"].total
            ent["graph"].replay()
            ops.launches += ent["launches"]
            return ent["logits"][:rows], ent["tokens"][:rows], ent["host_tokens"][:rows]
        sitems = [cache.host.StepItem(int(s), list(t), list(w)) for s, t, w in items]
        width = -(-self.max_context // min(cache.group_page_size))
        lay = cache.manager.plan_layout(sitems, width, padded)
        meta = torch.zeros(lay.total, dtype=torch.int32, device=self.rt.device)
        batch = cache.batch_from_layout(lay, meta)
        batch.max_kv_len = bucket
        cache.fill_metadata(sitems, lay, meta)
        logits = self.model.step(batch, cache)
        tokens = ops.argmax(logits)
        torch.cuda.synchronize()
        t_rec = time.perf_counter()
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        graph = torch.cuda.CUDAGraph()
        before = ops.launches
        stage = torch.empty(lay.total, dtype=torch.int32).pin_memory()
        host_tokens = torch.empty(padded, dtype=torch.int32).pin_memory()
        with torch.cuda.graph(graph, pool=self._graph_pool):
            meta.copy_(stage, non_blocking=True)
            g_logits = self.model.step(batch, cache)
            g_tokens = ops.argmax(g_logits)
            host_tokens.copy_(g_tokens, non_blocking=True)
        self.graphs_recorded += 1
        self.graph_record_seconds += time.perf_counter() - t_rec
        while len(self._graphs) >= self.max_graphs:
            self._graphs.popitem(last=False)
        self._graphs[key] = dict(graph=graph, layout=lay, meta=meta, logits=g_logits, tokens=g_tokens,
                                 launches=ops.launches - before, width=width, stage=stage, host_tokens=host_tokens)
        return logits[:rows], tokens[:rows], None

    # ------------------------------------------------------------- generation
    def submit(self, prompt: Iterable[int], params: SamplingParams | None = None, max_new_tokens: int = 16,
               eos_token=None) -> int:
        prompt = [int(t) for t in prompt]
        rid = self._next_id
        self._next_id += 1
        eos = [] if eos_token is None else ([int(eos_token)] if isinstance(eos_token, int) else [int(t) for t in eos_token])
        self.scheduler.submit(rid, prompt, int(max_new_tokens), eos)
        self._samplers[rid] = RequestSampler(params or SamplingParams(), prompt)
        return rid

    def abort(self, rid: int) -> bool:
        return self.scheduler.abort(rid)

    def _deliver(self, finished) -> None:
        for f in finished:
            self._results[f.id] = list(f.output)
            self._reasons[f.id] = f.reason
            self._samplers.pop(f.id, None)

    def run_step(self) -> list[tuple[int, int]]:
        """One scheduler tick: plan, run, sample, commit.  Returns ``(request id, token)`` for
        every token produced."""
        sched = self.scheduler
        plan = sched.plan()
        pitems = plan.items          # (a copy of the plan's list: taken once)
        if not pitems:
            fin = sched.drain_finished()
            self._deliver(fin)
            if not fin and not plan.preempted and sched.has_work():
                raise RuntimeError("the scheduler could not place any request")
            return []
        items, rows, pure_decode = [], [], True
        for it in pitems:
            toks = it.tokens
            if it.start == 0:
                self.cache.reset_state(it.slot)
            if it.sample:
                rows.append(it)
                items.append((it.slot, toks, [len(toks) - 1]))
            else:
                items.append((it.slot, toks, []))
            pure_decode = pure_decode and it.sample and len(toks) == 1
        samplers = [self._samplers[it.id] for it in rows]
        if self.use_graphs and pure_decode:
            logits, greedy, on_host = self._run_decode(items)
            if all(s.params.plain_greedy for s in samplers):
                if on_host is not None:
                    torch.cuda.current_stream().synchronize()
                    tokens = on_host.tolist()
                else:
                    tokens = greedy.tolist()
            else:
                tokens = sample_rows(self.rt.ops, logits, samplers)
        else:
            logits = self._run(items)
            tokens = sample_rows(self.rt.ops, logits, samplers)
        self.last_logits = logits
        self.rt.ops.check_errors()
        for smp, tok in zip(samplers, tokens):
            smp.note(tok)
        self._deliver(sched.commit(plan, tokens))
        return [(it.id, tok) for it, tok in zip(rows, tokens)]

    def run(self) -> None:
        while self.scheduler.has_work():
            self.run_step()

    def result(self, rid: int) -> list[int]:
        return self._results.pop(rid)

    def generate(self, prompts, max_new_tokens: int = 16, eos_token=None, temperature: float = 0.0,
                 top_p: float = 1.0, top_k: int = 0, min_p: float = 0.0, repetition_penalty: float = 1.0,
                 seed: int = 0):
        """Generates for one prompt (a list of token ids -> a list of token ids) or several
        (a list of lists -> a list of lists).  Every request uses ``seed`` for its own
        generator, so a prompt's output does not depend on what it was batched with."""
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        plist = [prompts] if single else list(prompts)
        params = SamplingParams(temperature=temperature, top_p=top_p, top_k=top_k, min_p=min_p,
                                repetition_penalty=repetition_penalty, seed=seed)
        ids = [self.submit(p, SamplingParams(**vars(params)), max_new_tokens, eos_token) for p in plist]
        self.run()
        failed = [i for i in ids if self._reasons.get(i) == "cache"]
        outs = [self.result(i) for i in ids]
        if failed:
            raise RuntimeError(f"{len(failed)} request(s) can never fit in the cache pool "
                               f"({self.cache.num_pages} pages of {self.cache.page_size} tokens)")
        return outs[0] if single else outs

    def stats(self) -> dict:
        st = self.scheduler.stats()
        pools = self.cache.stats()
        return {"steps": st.steps, "prompt_tokens": st.prompt_tokens, "decode_tokens": st.decode_tokens,
                "preemptions": st.preemptions, "finished": st.finished,
                "graphs_recorded": self.graphs_recorded, "graph_record_seconds": round(self.graph_record_seconds, 3),
                "eager_steps": self.eager_steps, "eager_launch_seconds": round(self.eager_launch_seconds, 3),
                "pages": [{"total": p.total_pages, "used": p.used_pages, "high_water": p.high_water} for p in pools]}


def generate(model_path: str, prompts, dtype="bfloat16", device="cuda:0", **kw):
    """Loads a model folder and generates (the shortest way from a folder to tokens)."""
    eng_kw = {k: kw.pop(k) for k in ("page_size", "num_pages", "max_tokens", "max_requests", "max_step_tokens",
                                     "max_context") if k in kw}
    return Engine.from_pretrained(model_path, dtype=dtype, device=device, **eng_kw).generate(prompts, **kw)
