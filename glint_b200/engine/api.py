"""The Python entry point, in the manner of the reference's ``glint.GlintLLM``
(src/python.rs:30-148): ``LLM(model_path).generate(prompt, max_tokens=256, temperature=0.0,
top_k=0, top_p=1.0, repeat_penalty=1.0, seed=None)`` returns only the newly generated tokens,
``model_info()`` returns the same dictionary, and errors surface as ``ValueError``.

This engine has no tokenizer (the reference's HF path refuses Gemma's SentencePiece
tokenizer.json anyway, src/model/tokenizer.rs:104-152): a prompt is a list of token ids and so
is the result.  A list of prompts is generated together by the continuous-batching scheduler.
"""
from __future__ import annotations

import torch

from ..errors import GlintError, RequestError
from ..sampling import DeviceSampler, SamplingParams
from .loading import build_engine, load_model, random_model
from .scheduler import Request, Scheduler


def default_cache_tokens(model, max_active, fraction=0.5):
    """Room for ``max_active`` requests at full context, limited to ``fraction`` of the device memory
    that is free now, and never below four contexts."""
    from ..cache import cache_bytes_per_token
    needs, cache_of = model.cache_needs()
    per_token = cache_bytes_per_token(needs, cache_of, torch.empty((), dtype=model.rt.dtype).element_size())
    free, _ = torch.cuda.mem_get_info(model.rt.device)
    fit = int(fraction * free) // max(per_token, 1)
    contexts = model.spec.max_positions
    return max(4 * contexts, min(max_active * contexts, fit))


class LLM:
    """A loaded model ready to generate.

    ``model_path``: folder with config.json and model.safetensors.  ``dtype``: 'bfloat16' (the
    serving kernels) or 'float32' (everything in true 32-bit).  ``cache_tokens``: how many
    tokens each cache group can hold in all (default: a full context for every running request, as
    far as half of the free device memory goes, and at least 4 contexts).  ``max_active``: requests
    running at a time.  ``max_step_tokens``: token budget of one step.  ``lookahead``: launch each
    decode step with the previous step's sampled tokens still on the device and read them one step
    late, so that the host's work overlaps the GPU's (same tokens as without it).
    """

    def __init__(self, model_path=None, dtype="bfloat16", device="cuda:0", cache_tokens=None, max_active=64,
                 max_step_tokens=2048, page_size=16, kernels="auto", model=None, lookahead=True):
        try:
            self.model = model if model is not None else load_model(model_path, dtype, device, kernels)
        except GlintError as e:
            raise ValueError(str(e)) from e
        spec = self.model.spec
        if cache_tokens is None:
            cache_tokens = default_cache_tokens(self.model, max_active)
        self.engine = build_engine(self.model, cache_tokens, num_slots=max_active, page_size=page_size)
        self.sampler = DeviceSampler(self.model.rt, spec.vocab_size, self.engine.cache)
        self.scheduler = Scheduler(self.engine, self.sampler, max_step_tokens=max_step_tokens,
                                   max_active=max_active, lookahead=lookahead)
        self.eos_token_id = spec.eos_token_id
        self._next_id = 0

    @classmethod
    def from_config(cls, config, seed=0, std=0.02, norm_std=0.1, dtype="bfloat16", device="cuda:0", **kw):
        """A model of ``config`` with random weights made on the device (no folder)."""
        return cls(model=random_model(config, seed, std, norm_std, dtype, device, kw.pop("kernels", "auto")),
                   **kw)

    def generate(self, prompt, max_tokens=256, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0,
                 seed=None, min_p=0.0, stop_at_eos=True):
        """Continue ``prompt`` (token ids) by up to ``max_tokens`` tokens; returns the new tokens.
        A list of prompts returns a list of results; with a seed, prompt ``i`` draws from
        ``seed + i``."""
        batch = len(prompt) > 0 and isinstance(prompt[0], (list, tuple))
        prompts = list(prompt) if batch else [prompt]
        requests = []
        try:
            vocab = self.model.spec.vocab_size
            for p in prompts:
                bad = [t for t in p if not 0 <= int(t) < vocab]
                if bad:
                    raise RequestError(f"token id {bad[0]} lies outside the vocabulary of {vocab}")
            for i, p in enumerate(prompts):
                params = SamplingParams(temperature=float(temperature), top_k=int(top_k), top_p=float(top_p),
                                        min_p=float(min_p), repeat_penalty=float(repeat_penalty),
                                        seed=None if seed is None else int(seed) + i)
                r = Request(self._next_id, [int(t) for t in p], int(max_tokens), params,
                            self.eos_token_id if stop_at_eos else None)
                self._next_id += 1
                self.scheduler.add(r)
                requests.append(r)
            self.scheduler.run()
            self.model.rt.check_status()
        except GlintError as e:
            for r in requests:            # leave no half-run request behind
                if not r.finished:
                    self.scheduler.abort(r)
            raise ValueError(str(e)) from e
        self.last_requests = requests
        out = [list(r.output) for r in requests]
        return out if batch else out[0]

    def model_info(self):
        return dict(self.model.spec.info)

    def cache_stats(self):
        return self.engine.cache.stats()


GlintLLM = LLM
