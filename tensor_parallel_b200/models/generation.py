"""Token generation for the self-contained models and their tensor-parallel wrappers:
greedy, nucleus (top-p) sampling and beam search, all with a KV cache that may be head-sharded
(``PerDeviceTensors``).  Works with anything callable as
``model(input_ids=..., past_key_values=..., use_cache=True) -> {logits, past_key_values}``.
Beam search reorders the cache per rank, on that rank's device (reference:
``src/tensor_parallel/pretrained_model.py:106-111``).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from tensor_parallel_b200.parallel.kv import PerDeviceTensors


def reorder_cache(past, beam_idx: torch.Tensor):
    def pick(entry):
        if isinstance(entry, PerDeviceTensors):
            return PerDeviceTensors(*(t.index_select(0, beam_idx.to(t.device)) for t in entry.tensors))
        if isinstance(entry, torch.Tensor):
            return entry.index_select(0, beam_idx.to(entry.device))
        return entry

    return tuple(tuple(pick(e) for e in layer) for layer in past)


@torch.no_grad()
def generate(model, input_ids: torch.Tensor, max_new_tokens: int = 20, num_beams: int = 1, do_sample: bool = False,
             top_p: float = 1.0, temperature: float = 1.0, eos_token_id: Optional[int] = None, output_scores: bool = False,
             generator: Optional[torch.Generator] = None, **model_kwargs):
    """Returns the generated ids ``[batch, prompt + new]`` (and the per-step score tensors when
    ``output_scores``: log-probabilities the next token was chosen from)."""
    if num_beams > 1:
        return _beam_search(model, input_ids, max_new_tokens, num_beams, eos_token_id, output_scores, model_kwargs)
    ids, past, scores = input_ids, None, []
    step_input = input_ids
    finished = torch.zeros(ids.shape[0], dtype=torch.bool, device=ids.device)
    for _ in range(max_new_tokens):
        out = model(input_ids=step_input, past_key_values=past, use_cache=True, **model_kwargs)
        past = out["past_key_values"]
        logits = out["logits"][:, -1].float().to(ids.device)
        if do_sample:
            logits = logits / temperature
            if top_p < 1.0:
                sorted_logits, order = logits.sort(descending=True)
                cum = sorted_logits.softmax(-1).cumsum(-1)
                drop = cum - sorted_logits.softmax(-1) > top_p
                sorted_logits = sorted_logits.masked_fill(drop, float("-inf"))
                logits = torch.full_like(logits, float("-inf")).scatter(1, order, sorted_logits)
            logprobs = logits.log_softmax(-1)
            nxt = torch.multinomial(logprobs.exp(), 1, generator=generator)[:, 0]
        else:
            logprobs = logits.log_softmax(-1)
            nxt = logprobs.argmax(-1)
        scores.append(logprobs)
        if eos_token_id is not None:
            nxt = torch.where(finished, torch.full_like(nxt, eos_token_id), nxt)
            finished |= nxt == eos_token_id
        ids = torch.cat([ids, nxt[:, None]], dim=1)
        step_input = nxt[:, None]
        if eos_token_id is not None and bool(finished.all()):
            break
    return (ids, scores) if output_scores else ids


def _beam_search(model, input_ids, max_new_tokens, num_beams, eos_token_id, output_scores, model_kwargs):
    batch, device = input_ids.shape[0], input_ids.device
    ids = input_ids.repeat_interleave(num_beams, dim=0)
    beam_scores = torch.zeros(batch, num_beams, device=device)
    beam_scores[:, 1:] = -1e9  # all beams start identical: keep only one alive
    past, step_input, scores = None, ids, []
    for _ in range(max_new_tokens):
        out = model(input_ids=step_input, past_key_values=past, use_cache=True, **model_kwargs)
        past = out["past_key_values"]
        logprobs = out["logits"][:, -1].float().to(device).log_softmax(-1)
        scores.append(logprobs)
        vocab = logprobs.shape[-1]
        total = (beam_scores.view(-1, 1) + logprobs).view(batch, num_beams * vocab)
        best, flat = total.topk(num_beams, dim=1)
        src_beam, token = flat // vocab, flat % vocab
        beam_idx = (src_beam + torch.arange(batch, device=device)[:, None] * num_beams).view(-1)
        ids = torch.cat([ids.index_select(0, beam_idx), token.view(-1, 1)], dim=1)
        beam_scores = best
        past = reorder_cache(past, beam_idx)
        step_input = token.view(-1, 1)
    best_rows = torch.arange(batch, device=device) * num_beams + beam_scores.argmax(dim=1)
    result = ids.index_select(0, best_rows)
    return (result, scores) if output_scores else result
