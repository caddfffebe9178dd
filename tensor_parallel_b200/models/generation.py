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
    if past is not None and not isinstance(past, (tuple, list)):
        # a stateful cache object (``transformers.Cache``): it reorders itself in place; under the single-process
        # runtime the call is mirrored to the other ranks' caches
        for method in ("reorder_cache", "batch_select_indices"):
            if hasattr(past, method):
                getattr(past, method)(beam_idx)
                return past
        raise TypeError(f"cannot reorder a cache of type {type(past).__name__} for beam search")

    def pick(entry):
        if isinstance(entry, PerDeviceTensors):
            return PerDeviceTensors(*(t.index_select(0, beam_idx.to(t.device)) for t in entry.tensors))
        if isinstance(entry, torch.Tensor):
            return entry.index_select(0, beam_idx.to(entry.device))
        return entry

    return tuple(tuple(pick(e) for e in layer) for layer in past)


@torch.no_grad()
def generate(model, input_ids: Optional[torch.Tensor] = None, max_new_tokens: int = 20, num_beams: int = 1, do_sample: bool = False,
             top_p: float = 1.0, temperature: float = 1.0, eos_token_id: Optional[int] = None, output_scores: bool = False,
             generator: Optional[torch.Generator] = None, inputs_embeds: Optional[torch.Tensor] = None, **model_kwargs):
    """Returns the generated ids ``[batch, prompt + new]`` (and the per-step score tensors when
    ``output_scores``: log-probabilities the next token was chosen from).  The prompt may be given as
    ``inputs_embeds [batch, prompt, hidden]`` instead of ids (the reference's ``test_generate_inputs_embeds`` case); the
    result then holds the new tokens only."""
    if (input_ids is None) == (inputs_embeds is None):
        raise ValueError("pass exactly one of input_ids / inputs_embeds")
    if num_beams > 1:
        return _beam_search(model, input_ids, max_new_tokens, num_beams, eos_token_id, output_scores, model_kwargs, inputs_embeds)
    prompt = input_ids if input_ids is not None else inputs_embeds
    ids = input_ids if input_ids is not None else torch.empty(prompt.shape[0], 0, dtype=torch.long, device=prompt.device)
    past, scores = None, []
    step_input = input_ids
    finished = torch.zeros(ids.shape[0], dtype=torch.bool, device=ids.device)
    for step in range(max_new_tokens):
        if step == 0 and inputs_embeds is not None:
            out = model(inputs_embeds=inputs_embeds, past_key_values=past, use_cache=True, **model_kwargs)
        else:
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


def _beam_search(model, input_ids, max_new_tokens, num_beams, eos_token_id, output_scores, model_kwargs, inputs_embeds=None):
    prompt = input_ids if input_ids is not None else inputs_embeds
    batch, device = prompt.shape[0], prompt.device
    if input_ids is not None:
        ids = input_ids.repeat_interleave(num_beams, dim=0)
    else:
        ids = torch.empty(batch * num_beams, 0, dtype=torch.long, device=device)
        inputs_embeds = inputs_embeds.repeat_interleave(num_beams, dim=0)
    beam_scores = torch.zeros(batch, num_beams, device=device)
    beam_scores[:, 1:] = -1e9  # all beams start identical: keep only one alive
    past, step_input, scores = None, ids, []
    for step in range(max_new_tokens):
        if step == 0 and inputs_embeds is not None:
            out = model(inputs_embeds=inputs_embeds, past_key_values=past, use_cache=True, **model_kwargs)
        else:
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
