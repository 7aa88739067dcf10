"""Philox stream bookkeeping for dropout.

Dropout draws element ``i`` of the flattened ``[B, Hq, M, N]`` probability tensor from Philox
counter ``offset + i`` under key ``seed``. Both numbers come from the default CUDA generator of the
device the call runs on, exactly as the reference does (``flag_attn/dropout.py:17-27``), so that a
caller who seeds ``torch.cuda.manual_seed`` gets the same mask from either implementation.
"""
from __future__ import annotations

import torch

_ALIGN = 4  # generator offsets advance in multiples of four draws


def _device_index(device) -> int:
    if device is None:
        return torch.cuda.current_device()
    if isinstance(device, torch.device):
        return torch.cuda.current_device() if device.index is None else device.index
    return int(device)


def reserve_philox_stream(num_draws: int, device=None) -> tuple[int, int]:
    """Reads ``(seed, offset)`` of the device's default generator and reserves ``num_draws``
    counters (rounded up to a multiple of four) by moving the generator's offset past them.

    Returns Python ints; a seed with the top bit set comes back negative, as a two's-complement
    int64, which is how the reference reports it too.
    """
    generator = torch.cuda.default_generators[_device_index(device)]
    state = generator.get_state()            # a copy: 16 bytes = (seed, offset) as int64
    words = state.view(torch.int64)
    seed, offset = int(words[0]), int(words[1])
    words[1] = offset + -(-int(num_draws) // _ALIGN) * _ALIGN
    generator.set_state(state)
    return seed, offset


def as_u64(value: int) -> int:
    """Two's-complement bit pattern of a Python int as an unsigned 64-bit value."""
    return int(value) & 0xFFFFFFFFFFFFFFFF
