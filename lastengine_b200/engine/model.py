"""A model: the parts a plan names, built through the registries, with their weights.

`forward` runs the schedule over the rows of a step and returns the logits of the wanted
rows.  It is the only forward pass in the library: generation, the replay program and the
benchmark all go through it.
"""
from __future__ import annotations

import torch

from .. import parts as _parts  # noqa: F401  (registers the built-in parts)
from ..parts.base import BuildEnv, ModelPlan, TensorSpec
from ..registry import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS


class Model:
    def __init__(self, plan: ModelPlan, env: BuildEnv):
        self.plan, self.env = plan, env
        self.embedding = EMBEDDINGS.get(plan.embedding.kind)(**plan.embedding.params)
        self.final_norm = NORMS.get(plan.final_norm.kind)(**plan.final_norm.params)
        self.head = HEADS.get(plan.head.kind)(**plan.head.params)
        self.blocks = []
        for ls in plan.layers:
            mixer = MIXERS.get(ls.mixer.kind)(**ls.mixer.params)
            ffn = FEED_FORWARDS.get(ls.ffn.kind)(**ls.ffn.params)
            norm = lambda s: None if s is None else NORMS.get(s.kind)(**s.params)  # noqa: E731
            self.blocks.append(BLOCKS.get(ls.block)(
                mixer=mixer, ffn=ffn, mixer_norm=norm(ls.mixer_norm), ffn_norm=norm(ls.ffn_norm),
                post_mixer_norm=norm(ls.post_mixer_norm), post_ffn_norm=norm(ls.post_ffn_norm)))
        self.hidden_size, self.vocab_size = plan.hidden_size, plan.vocab_size

    # ---- tensors ------------------------------------------------------------------------
    def named_parts(self) -> list[tuple[str, object]]:
        """(tensor-name prefix, part) for every part that may own tensors."""
        n = self.plan.names
        out = [(n.get("embedding", "embedding"), self.embedding),
               (n.get("final_norm", "final_norm"), self.final_norm),
               (n.get("head", "head"), self.head)]
        for ls, blk in zip(self.plan.layers, self.blocks):
            for role, part in blk.parts().items():
                out.append((f"{ls.prefix}.{ls.names.get(role, role)}", part))
        return out

    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs: dict[str, TensorSpec] = {}
        for prefix, part in self.named_parts():
            for rel, spec in part.tensors().items():
                name = spec.shared_name or f"{prefix}.{rel}"
                if name in specs and specs[name] != spec:
                    raise ValueError(f"tensor '{name}' is declared twice, as {specs[name]} and as {spec}")
                specs[name] = spec
        return specs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        """`tensors`: canonical name -> tensor on the device in the dtype of its role."""
        for prefix, part in self.named_parts():
            own = {}
            for rel, spec in part.tensors().items():
                name = spec.shared_name or f"{prefix}.{rel}"
                if name in tensors:
                    own[rel] = tensors[name]
            part.load(own, self.env)
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding)

    def cache_specs(self) -> dict[int, object]:
        """cache entry id -> spec, for the entries that own storage."""
        specs = {}
        for i, e in enumerate(self.plan.schedule):
            if e.cache is None or e.cache == i:
                specs[i] = self.blocks[e.layer].mixer.cache_spec()
        return specs

    # ---- the forward pass ---------------------------------------------------------------
    def forward(self, batch, cache) -> torch.Tensor:
        """Runs the step's rows through every scheduled layer; returns float logits
        [batch.n_logit_rows, vocab] (a view of workspace memory, valid until the next step)."""
        env, ws = self.env, self.env.workspace
        M, D = batch.n_rows, self.hidden_size
        x = ws.get("model.x", (M, D), torch.float32)
        self.embedding.forward(x, batch.tokens)
        sched = self.plan.schedule
        pending = None      # the half of the next block's first norm that the last block left (decode steps)
        for i, e in enumerate(sched):
            entry = i if e.cache is None else e.cache
            view = cache.view(entry, e.writes_cache and entry == i, batch.tables)
            block = self.blocks[e.layer]
            after = self.blocks[sched[i + 1].layer] if i + 1 < len(sched) else None
            # (norm, part that reads it) of the block that runs next, for blocks that can split a norm
            env.next_block_norm = after.first_reader() if hasattr(after, "first_reader") else None
            if pending is not None:
                pending = block.forward(x, batch, view, env, pending=pending)
            else:
                pending = block.forward(x, batch, view, env)
        env.next_block_norm = None
        R = batch.n_logit_rows
        logits = ws.get("model.logits", (R, self.vocab_size), torch.float32)
        if R:
            xn = ws.get("model.xn", (R, D), env.dtype)
            self.final_norm.forward(xn, x, rows=batch.logit_rows)
            self.head.forward(logits, xn)
        return logits
