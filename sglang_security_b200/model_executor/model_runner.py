"""ModelRunner: owns the model, the token pool, the page allocator, the request table and the state
pool of one GPU, and runs one engine step over them (the reference's ModelRunner,
python/sglang/srt/model_executor/model_runner.py: init_memory_pool + forward)."""
from __future__ import annotations

from typing import List, Optional

import torch

from ..configs.model_config import ModelConfig
from ..managers.schedule_batch import Req, StepItem, prepare
from ..mem_cache.latent_pool import LatentTokenToKVPool, SeqStatePool
from ..mem_cache.memory_pool import ReqToTokenPool
from ..mem_cache.paged_allocator import PagedTokenToKVPoolAllocator
from ..model_loader.loader import load_model

PAGE_SIZE = 64


class ModelRunner:
    def __init__(self, model_path: str, dtype: torch.dtype = torch.bfloat16, max_total_tokens: int = 8192,
                 max_running_requests: int = 4, context_length: Optional[int] = None,
                 device: str = "cuda", page_size: int = PAGE_SIZE, model=None, model_config=None):
        if not torch.cuda.is_available():
            raise RuntimeError("ModelRunner needs a CUDA device (there is no CPU path)")
        if dtype == torch.float32:
            # true 32-bit products: no reduced-precision matrix mode
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
        self.device, self.dtype, self.page_size = device, dtype, page_size
        self.model_config = model_config or ModelConfig(model_path)
        self.model = model if model is not None else load_model(self.model_config, device, dtype)
        pages = (max_total_tokens + page_size - 1) // page_size
        self.max_total_tokens = pages * page_size
        self.context_length = context_length or self.max_total_tokens
        # a model with a table of learned positions cannot run past it
        limit = getattr(self.model, "max_positions", None)
        if limit:
            self.context_length = min(self.context_length, int(limit))
        self.max_running_requests = max_running_requests
        spec = self.model.cache_spec()
        if spec.kind not in ("latent", "rows"):
            raise ValueError(f"cache kind {spec.kind!r} is not served by this runner")
        self.req_to_token_pool = ReqToTokenPool(max_running_requests, self.context_length, device)
        self.token_to_kv_pool = LatentTokenToKVPool(self.max_total_tokens, page_size, dtype,
                                                    spec.row_dims, spec.source_of, device,
                                                    block_summaries=spec.block_summaries)
        self.allocator = PagedTokenToKVPoolAllocator(self.max_total_tokens, page_size, dtype, device,
                                                     kvcache=self.token_to_kv_pool)
        self.state_pool = SeqStatePool(max_running_requests, spec.state_widths, device)

    # ---- request slots ---------------------------------------------------------------------------
    def admit(self, req: Req) -> bool:
        slots = self.req_to_token_pool.alloc(1)
        if slots is None:
            return False
        req.req_pool_idx, req.cached_len = slots[0], 0
        return True

    def release(self, req: Req) -> None:
        if req.req_pool_idx is None:
            return
        if req.cached_len:
            self.allocator.free(self.req_to_token_pool.req_to_token[req.req_pool_idx, :req.cached_len]
                                .to(torch.int64))
        self.req_to_token_pool.free(req.req_pool_idx)
        req.req_pool_idx = None

    def free_token_slots(self) -> int:
        return self.allocator.available_size()

    def pages_needed(self, req: Req, new_tokens: int) -> int:
        have = (req.cached_len + self.page_size - 1) // self.page_size
        need = (req.cached_len + new_tokens + self.page_size - 1) // self.page_size
        return need - have

    # ---- one step --------------------------------------------------------------------------------
    @torch.inference_mode()
    def forward(self, items: List[StepItem], layer_hook=None) -> Optional[torch.Tensor]:
        """Runs the new tokens of every item as one batch.  -> logits [wanted rows, vocab] in the
        order of the items and of their `want` lists (None if nothing is wanted)."""
        fb = prepare(items, self.req_to_token_pool, self.allocator, self.token_to_kv_pool,
                     self.state_pool, self.device)
        if layer_hook is not None:
            fb.extra["layer_hook"] = layer_hook
        hidden = self.model(fb.extra["input_ids"], fb)
        rows, start = [], 0
        for it in items:
            rows += [start + w for w in it.want]
            start += len(it.tokens)
        if not rows:
            return None
        idx = torch.tensor(rows, dtype=torch.int64).to(self.device, non_blocking=True)
        return self.model.compute_logits(hidden[idx])
