"""Trace replay over the engine's own model, step function, cache and kernels."""
from __future__ import annotations

from typing import Optional

import torch

from . import ops
from .cache.manager import CacheManager
from .engine.loading import load_model
from .engine.runner import ModelRunner, StepEntry


class Replay:
    """Holds a loaded model and a cache pool of ``max_tokens`` tokens; ``run_step`` feeds
    one step record.  It has no forward pass, cache or loader of its own: it is the
    runner that generation uses, driven by given tokens instead of sampled ones."""

    def __init__(self, model_dir: str, dtype: str, max_tokens: int, page_size: int = 16, max_running: int = 8,
                 device: str = "cuda:0"):
        if not torch.cuda.is_available():
            raise RuntimeError("trace replay needs a CUDA device: the engine has no CPU path")
        torch.cuda.set_device(device)
        self.config, self.model = load_model(model_dir, dtype, device)
        num_pages = max(1, -(-int(max_tokens) // page_size))
        self.cache = CacheManager(self.model.cache_needs(), page_size, num_pages, max_running, self.model.dtype, device)
        self.runner = ModelRunner(self.model, self.cache, device)

    def run_step(self, record: dict) -> Optional[torch.Tensor]:
        """Run one ``{"step", "entries", "end"}`` record; returns the wanted logits on the
        host (float32 ``[wanted, vocab]``) or None when nothing was wanted."""
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in record.get("entries", [])]
        out = None
        if entries:
            logits = self.runner.step(entries)
            if logits.shape[0]:
                out = logits.cpu()
            else:
                torch.cuda.current_stream().synchronize()
            ops.check_wait_words()          # a kernel that gave up a bounded wait must not pass for a result
        for rid in record.get("end", []):
            if self.cache.has(rid):
                self.runner.finish(rid)
        return out
