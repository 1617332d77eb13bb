"""What the decoder families with an fp32 residual stream and ragged steps share on top of their layer stacks: the vocabulary head,
the cache manager they ask for (block pool + state slots, utils/paged.py `HybridCacheManager`), the flash families' forward
signature over a `RaggedStep`, and the fused greedy step protocol of `FlashCausalLM._decode_fused_greedy`.

A family subclasses `RaggedDecoderForCausalLM` and gives it `self.model`: a module with `layers` (each with a `.mixer` that has
`cache_spec()`), `final_norm`, `kv_cache_manager`, and `forward(input_ids, step, max_s) -> fp32 stream [T, width]` (or whatever its `final_norm` takes
per token row: a family with several streams returns [T, streams, width]).
"""
from __future__ import annotations

import os
from typing import Optional

import torch
from torch import nn

from ... import ops_seq as ops
from ...utils.paged import HybridCacheManager, PagedKVState
from .python_step import PythonStep, _NoScratch


class _HeadView:
    """what FlashCausalLM reads on a model's vocabulary head: `.linear.weight` and `.should_gather`"""

    def __init__(self, weight):
        self.linear, self.should_gather = self, False
        self.weight = weight


class RaggedDecoderForCausalLM(nn.Module):
    ragged_steps = True           # FlashCausalLM.step_ragged: any mix of prompts, portions and decoded tokens in one batch
    logits_dtype = torch.float32
    scratch = _NoScratch()        # nothing of the fused step is ever re-allocated
    logit_scale = 1.0             # logits = head(final_norm(x)) * logit_scale

    @property
    def fused_greedy_enabled(self) -> bool:
        """plain greedy decode of a stable batch runs as one CUDA graph (decode_advance + this forward + arg-max + the batch's
        bookkeeping), as for the other Python-driven families; B200_PY_FUSED_STEP=0 keeps it op by op"""
        return os.environ.get("B200_PY_FUSED_STEP", "") != "0"

    def __init__(self, config, weights, model: nn.Module, head_tensor: str = "head"):
        """`head_tensor`: the checkpoint tensor of the vocabulary head ("embed" for a family whose embedding table is its head)"""
        super().__init__()
        self.config = config
        self.process_group = weights.process_group
        self.device = torch.device(weights.device)
        self.dtype = weights.dtype
        self.model = model
        self.head = model.embed if head_tensor == "embed" and hasattr(model, "embed") else weights.get_tensor(head_tensor).contiguous()
        self.lm_head = _HeadView(self.head)

    @property
    def kv_cache_manager(self):
        return self.model.kv_cache_manager

    @kv_cache_manager.setter
    def kv_cache_manager(self, manager):
        self.model.kv_cache_manager = manager

    def get_input_embeddings(self):
        return None  # prompt-tuning prefixes are not defined for these families (token ids are needed past the embedding)

    def prepare_positions(self, max_s: int) -> None:
        """grows whatever per-position tables the layers keep, so that nothing is allocated inside a captured graph"""
        for layer in self.model.layers:
            if hasattr(layer.mixer, "prepare_positions"):      # a mixer with several tables, or with mixers of its own
                layer.mixer.prepare_positions(int(max_s) + 1, self.device)
            elif getattr(layer.mixer, "rotary", None) is not None:
                layer.mixer.rotary.tables(int(max_s) + 1, self.device)

    def make_cache_manager(self, dtype, device, num_blocks: Optional[int], num_state_slots: Optional[int]) -> HybridCacheManager:
        specs = [layer.mixer.cache_spec() for layer in self.model.layers]
        slots = int(num_state_slots or 64)
        if num_blocks is None:
            per_block = sum(16 * s.row_width for s in specs if s.kind == "paged") * torch.empty(0, dtype=dtype).element_size()
            free, _ = torch.cuda.mem_get_info(device)
            num_blocks = max(int(free * 0.6) // max(per_block, 1), 1) if per_block else 1
            num_blocks = min(num_blocks, 1 << 22)
        return HybridCacheManager(specs, dtype, device, int(num_blocks), slots)

    # ---- the fused greedy step protocol of FlashCausalLM._decode_fused_greedy (python_step.py)
    def make_step(self, *, T: int, B: int, is_prefill: bool, max_s: int, input_ids, position_ids, kv: PagedKVState, cu_seqlens=None,
                  head_rows=None, logits=None, next_ids=None, inputs_embeds=None) -> PythonStep:
        if is_prefill or head_rows is not None or inputs_embeds is not None or T != B:
            raise NotImplementedError("the fused step is decode-only")
        self.prepare_positions(max_s)
        cu_q = torch.arange(B + 1, dtype=torch.int32, device=self.device)
        return PythonStep(T=T, B=B, max_s=int(max_s) + 1, input_ids=input_ids, position_ids=position_ids, kv=kv, logits=logits,
                          next_ids=next_ids, banned=None, decode_marker=cu_q)

    def run_step(self, s: PythonStep) -> None:
        logits, _ = self.forward(s.input_ids, s.position_ids, None, s.decode_marker, s.max_s, None, s.kv)
        s.logits.copy_(logits)
        if s.next_ids is not None:
            lg = s.logits
            if s.banned is not None:  # per-row banned id of the arg-max (min_new_tokens EOS mask); -1 bans nothing
                ids = torch.arange(lg.shape[1], device=lg.device)
                lg = lg.masked_fill(ids[None, :] == s.banned[:, None], float("-inf"))
            torch.argmax(lg, dim=-1, out=s.next_ids)

    def forward(self, input_ids, position_ids, cu_seqlens, cu_seqlens_q, max_s, inputs_embeds: Optional[torch.Tensor] = None,
                past_key_values: Optional[PagedKVState] = None, pre_allocate_past_size: Optional[int] = None,
                lm_head_indices: Optional[torch.Tensor] = None):
        """Flash-family signature.  `cu_seqlens_q` None: every sequence brings its whole prompt (`cu_seqlens` are the row
        boundaries); otherwise `cu_seqlens_q` are the row boundaries of this step and each sequence's rows continue at
        `position_ids`.  -> (fp32 logits of the rows `lm_head_indices` (all rows when None), past_key_values)."""
        if inputs_embeds is not None:
            raise NotImplementedError("inputs_embeds: these families take token ids")
        kv = past_key_values
        if kv is None or kv.state_slots is None:
            raise ValueError("past_key_values must be a PagedKVState of the model's HybridCacheManager")
        cu_q = (cu_seqlens if cu_seqlens_q is None else cu_seqlens_q).to(torch.int32)
        T, B = input_ids.shape[0], cu_q.shape[0] - 1
        if T == B:  # one row per sequence
            seq_of_token = torch.arange(B, dtype=torch.int32, device=cu_q.device)
        else:
            counts = cu_q[1:] - cu_q[:-1]
            seq_of_token = torch.repeat_interleave(torch.arange(B, dtype=torch.int32, device=cu_q.device), counts.to(torch.int64),
                                                   output_size=T)
        step = ops.RaggedStep(T=T, B=B, position_ids=position_ids.contiguous(), cu_q=cu_q.contiguous(), seq_of_token=seq_of_token.contiguous(),
                              slot_mapping=kv.slot_mapping[:T].contiguous(), block_table=kv.block_table, state_slots=kv.state_slots)
        x = self.model(input_ids.contiguous(), step, int(max_s))
        if lm_head_indices is not None:
            x = x[lm_head_indices].contiguous()
        logits = ops.linear(self.model.final_norm(x), self.head, out_dtype=torch.float32)
        if self.logit_scale != 1.0:
            logits.mul_(self.logit_scale)
        return logits, kv
