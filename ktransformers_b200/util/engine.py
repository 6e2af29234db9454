"""Engine — the generation entry point for step-function models: model + paged cache + scheduler + sampler.

    step(entries, end)    run one ragged batch of (sequence id, next tokens, wanted rows) through the model's step function
                          against the cache and state earlier steps left; returns fp32 logits of the wanted rows
    generate(prompts)     continuous batching: the scheduler cuts prompts into portions and mixes them with decode tokens,
                          the sampler picks each next token

(The reference's single-stream loop is `prefill_and_generate`, archive/ktransformers/util/utils.py:345-560: chunked prefill,
then a decode loop over a static cache with a sampler from the generation config.)"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .scheduler import Request, Scheduler


class Sampler:
    """Greedy when temperature == 0, else temperature / top-k / top-p sampling (fp32 logits on the device)."""

    def __init__(self, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, seed: Optional[int] = None):
        self.temperature, self.top_k, self.top_p = temperature, top_k, top_p
        self.generator = None
        if seed is not None and torch.cuda.is_available():
            self.generator = torch.Generator(device="cuda")
            self.generator.manual_seed(seed)

    def __call__(self, logits: torch.Tensor) -> torch.Tensor:
        if self.temperature <= 0.0:
            return logits.argmax(-1)
        z = logits / self.temperature
        if self.top_k and self.top_k < z.shape[-1]:
            kth = z.topk(self.top_k, -1).values[..., -1:]
            z = z.masked_fill(z < kth, float("-inf"))
        p = torch.softmax(z, -1)
        if self.top_p < 1.0:
            sp, si = p.sort(-1, descending=True)
            drop = sp.cumsum(-1) - sp > self.top_p
            sp = sp.masked_fill(drop, 0.0)
            p = torch.zeros_like(p).scatter_(-1, si, sp)
            p = p / p.sum(-1, keepdim=True)
        return torch.multinomial(p, 1, generator=self.generator).squeeze(-1)


class _CapturedStep:
    """A decode step of a fixed batch size as a CUDA graph: static index / token buffers in, logits of every row out."""

    def __init__(self, model, cache, n: int):
        from ..models.custom_cache import ForwardBatch
        dev = cache.device
        self.meta = torch.zeros((ForwardBatch.N_META, n), dtype=torch.int32, device=dev)
        self.tokens = torch.zeros(n, dtype=torch.int64, device=dev)
        self.all_rows = torch.arange(n, dtype=torch.int64, device=dev)
        self.graph, self.logits = None, None

    def capture(self, model, cache):
        from ..models.custom_cache import ForwardBatch
        batch = ForwardBatch(self.meta, self.tokens, self.all_rows, cache.capacity_per_sequence(), self.meta.shape[1])
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = model(batch, cache)


class Engine:
    """`cuda_graphs`: steps in which every sequence brings exactly one token (decode) replay a captured graph per batch size
    after two eager steps of that size (the launch-bound inner loop of generation); everything else runs eagerly."""

    graph_max_batch = 47        # below the experts' and the router's switch to their prompt-sized paths

    def __init__(self, model, max_tokens: int = 8192, max_slots: int = 8, page_size: int = 64, max_step_tokens: int = 2048, cuda_graphs: bool = True):
        self.model = model
        self.cache = model.make_cache(max_tokens, max_slots=max_slots, page_size=page_size)
        self.scheduler = Scheduler(self.cache, max_step_tokens=max_step_tokens)
        self.cuda_graphs = cuda_graphs and self.cache.device.type == "cuda" and getattr(model, "decode_is_capturable", lambda n: True)(self.graph_max_batch)
        self._captured, self._seen = {}, {}

    @torch.no_grad()
    def step(self, entries: Sequence, end: Sequence = ()) -> torch.Tensor:
        """entries: (sequence id, tokens, wanted places among these tokens).  Sequences named in `end` give their pages, slot
        and state back after the step."""
        n = len(entries)
        if self.cuda_graphs and n <= self.graph_max_batch and all(len(e[1]) == 1 for e in entries):
            self._seen[n] = self._seen.get(n, 0) + 1
            if self._seen[n] > 2:
                logits = self._replay(entries)
                self.cache.commit()
                for seq_id in end:
                    self.cache.close(seq_id)
                return logits
        batch = self.cache.build_batch(entries)
        logits = self.model(batch, self.cache)
        self.cache.commit()
        for seq_id in end:
            self.cache.close(seq_id)
        return logits

    def _replay(self, entries) -> torch.Tensor:
        n = len(entries)
        step = self._captured.get(n)
        if step is None:
            step = self._captured[n] = _CapturedStep(self.model, self.cache, n)
        batch = self.cache.build_batch(entries, static=(step.meta, step.tokens))
        if step.graph is None:
            torch.cuda.current_stream().synchronize()
            step.capture(self.model, self.cache)
        step.graph.replay()
        return step.logits.index_select(0, batch.want)

    @torch.no_grad()
    def generate(self, prompts: List[List[int]], max_new_tokens: int, sampler: Optional[Sampler] = None, stop_token: Optional[int] = None) -> List[List[int]]:
        sampler = sampler or Sampler()
        reqs = [Request(("gen", i), list(p), max_new_tokens) for i, p in enumerate(prompts)]
        for r in reqs:
            self.scheduler.add(r)
        while self.scheduler.has_work():
            entries = self.scheduler.schedule()
            if not entries:
                raise MemoryError("the scheduler cannot place any request: the cache is too small for the oldest prompt")
            logits = self.step([(e.request.id, e.tokens, [len(e.tokens) - 1] if e.want_last else []) for e in entries])
            picked = sampler(logits).tolist() if logits.shape[0] else []
            k = 0
            for e in entries:
                r = e.request
                if r.prefilling:
                    r.fed += len(e.tokens)
                if not e.want_last:
                    continue
                tok = picked[k]
                k += 1
                r.output.append(tok)
                r.pending = tok
                if len(r.output) >= r.max_new_tokens or (stop_token is not None and tok == stop_token):
                    self.scheduler.finish(r)
        return [r.output for r in reqs]
