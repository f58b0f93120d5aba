"""lastengine_b200: a small single-GPU model library with generation for the LFM3 hybrid
decoder, on hand-written sm_100a kernels.

    from lastengine_b200 import Engine, SamplingParams
    eng = Engine.from_pretrained("model_dir", dtype="bfloat16", max_tokens=65536)
    out = eng.generate([[1, 2, 3], [4, 5]], SamplingParams(temperature=0.0), max_new_tokens=16)
    out.tokens, out.finish_reasons, out.stats
"""
from __future__ import annotations

from typing import Sequence

from .config import ConfigError  # noqa: F401
from .engine.engine import Engine, EngineOptions, StepError  # noqa: F401
from .engine.generate import GenerationLoop, GenerationResult, GenerationStats  # noqa: F401
from .sampling.params import SamplingParams  # noqa: F401

__version__ = "0.1.0"


def generate(engine: Engine, prompts: Sequence[Sequence[int]], sampling: SamplingParams | None = None,
             max_new_tokens: int = 128, stop_token_ids: Sequence[int] | None = None,
             max_batch: int = 64, max_seq_len: int | None = None, use_graphs: bool | None = None) -> GenerationResult:
    """Generates for every prompt (lists of token ids), batch after batch.

    `stop_token_ids` defaults to the model's `eos_token_id`; a stop token ends its request and
    is not part of the output.  `use_graphs` and a sampling seed that the call leaves open come
    from the engine's options.
    """
    import dataclasses
    from .engine.generate import EngineBackend
    sampling = sampling or SamplingParams()
    if sampling.seed is None and engine.options.seed is not None:
        sampling = dataclasses.replace(sampling, seed=engine.options.seed)
    if use_graphs is None:
        use_graphs = engine.options.use_graphs
    stops = tuple(stop_token_ids) if stop_token_ids is not None else tuple(engine.plan.eos_token_ids)
    backend = None
    if use_graphs:
        try:
            from .engine.graph import GraphBackend
            backend = GraphBackend(engine, sampling, max_batch=max_batch, max_seq_len=max_seq_len)
        except ImportError:
            backend = None
    if backend is None:
        backend = EngineBackend(engine, sampling)
    loop = GenerationLoop(backend, sampling, max_new_tokens, stops, max_batch=max_batch,
                          max_seq_len=max_seq_len or engine.max_tokens + 1,
                          token_budget=engine.cache.n_pages * engine.cache.page_size,
                          page=engine.cache.page_size)
    res = loop.run(prompts)
    res.backend = backend
    return res


Engine.generate = lambda self, prompts, sampling=None, **kw: generate(self, prompts, sampling, **kw)
