"""Dense position / mask inputs of the classic (non-paged) decoder graph, kept for API parity.

The paged runtime needs neither: positions are packed per token and the attention kernel reads lengths, not masks.  Callers
that drive an exported graph with `position_ids` / `attention_mask` inputs (and tests that compare against such a graph)
get the reference's update rules here (src/cpu/interface.cpp:108-167, src/cuda/model_kernels.cu:17-84) as tensor functions
that work on CPU and CUDA tensors alike.
"""
from __future__ import annotations

import torch


def initial_position_ids_and_mask(input_ids: torch.Tensor, pad_token_id: int):
    """[batch, seq] ids -> (position_ids, attention_mask): pads get mask 0 and position 0, real tokens count from 0
    (the positions a left- or right-padded prompt starts with, src/models/position_inputs.cpp)."""
    mask = (input_ids != pad_token_id).to(input_ids.dtype)
    pos = (torch.cumsum(mask, dim=1) - 1).clamp(min=0) * mask
    return pos.to(input_ids.dtype), mask


def update_position_ids(position_ids: torch.Tensor, batch_beam_size: int, total_length: int, new_kv_length: int) -> torch.Tensor:
    """One row: the positions of the `new_kv_length` tokens being fed are total_length - new_kv_length .. total_length - 1
    (continuous decoding).  Several rows: each row's single position advances by one."""
    if batch_beam_size == 1:
        return torch.arange(total_length - new_kv_length, total_length, dtype=position_ids.dtype, device=position_ids.device).reshape(1, -1)
    return position_ids + 1


def update_attention_mask(mask: torch.Tensor, batch_beam_size: int, total_length: int) -> torch.Tensor:
    """[rows, total_length - 1] -> [rows, total_length]: the previous columns (a row of ones when there is one row: no padding
    is assumed there) and a 1 for the new token."""
    if batch_beam_size == 1:
        return torch.ones(1, total_length, dtype=mask.dtype, device=mask.device)
    return torch.cat([mask[:, : total_length - 1], torch.ones(mask.shape[0], 1, dtype=mask.dtype, device=mask.device)], dim=1)


def update_attention_mask_static(mask: torch.Tensor, new_kv_length: int, total_length: int) -> torch.Tensor:
    """Share-buffer form: a [rows, max_length] mask updated in place, columns total_length - new_kv_length .. total_length - 1
    become 1."""
    mask[:, total_length - new_kv_length: total_length] = 1
    return mask
