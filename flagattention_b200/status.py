"""Device status word of the CUDA kernels, and how the host gets to hear of it.

Every wait inside the kernels is bounded: a wait that does not complete records a code in a
per-device ``int32`` word (passed to every launch) and the CTA leaves with its TMEM released. The
outputs of such a launch are incomplete, so the operators must not let it pass unnoticed, yet none of
them may synchronise (they launch asynchronously on the caller's stream, as the reference's do).

``poll(device)`` is what every operator calls before it launches: it looks, without blocking, at the
last copy of the word that has reached pinned host memory and raises if a kernel reported a failure;
when no copy is in flight and the previous one is older than ``POLL_INTERVAL_S`` it enqueues the next
copy (one ``cudaMemcpyAsync`` and one event record on the caller's stream). A failure therefore
surfaces at one of the next operator calls after the failing launch has finished.
``check_device_status`` is the synchronous form for tests, benchmarks and anyone about to trust a result.
"""
from __future__ import annotations

import time

import torch

__all__ = ["status_word", "poll", "check_device_status", "known_devices", "POLL_INTERVAL_S"]

POLL_INTERVAL_S = 0.05

CODE_NAMES = {1: "TMA load never arrived", 2: "MMA never completed", 3: "softmax group never arrived",
              4: "ring slot never freed"}


class _DeviceStatus:
    __slots__ = ("word", "host", "event", "pending", "last_poll")

    def __init__(self, device: torch.device):
        self.word = torch.zeros(1, dtype=torch.int32, device=device)
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event = torch.cuda.Event()
        self.pending = False
        self.last_poll = 0.0


_devices: dict[int, _DeviceStatus] = {}


def _index(device) -> int:
    if device is None:
        return torch.cuda.current_device()
    device = torch.device(device)
    return device.index if device.index is not None else torch.cuda.current_device()


def _state(device) -> _DeviceStatus:
    idx = _index(device)
    st = _devices.get(idx)
    if st is None:
        st = _devices[idx] = _DeviceStatus(torch.device("cuda", idx))
    return st


def status_word(device) -> torch.Tensor:
    """The device's status word (one int32, zero while every wait has completed)."""
    return _state(device).word


def known_devices() -> list[int]:
    """Ordinals of the devices this process has launched kernels on."""
    return sorted(_devices)


def _raise(code: int, st: _DeviceStatus):
    st.word.zero_()
    st.host.zero_()
    what = CODE_NAMES.get(code, "unknown wait")
    raise RuntimeError(f"b200attn kernel reported device-side wait timeout (code {code}: {what}); the "
                       "results of the launches since the last check are incomplete")


def poll(device) -> torch.Tensor:
    """Non-blocking look at the status word (see the module docstring); returns the word so that a
    caller can pass its address to the next launch."""
    st = _state(device)
    now = time.monotonic()
    if not st.pending and now - st.last_poll < POLL_INTERVAL_S:
        return st.word
    if torch.cuda.is_current_stream_capturing():
        return st.word                      # nothing here may enter a CUDA graph
    if st.pending:
        if not st.event.query():
            return st.word
        st.pending = False
        code = int(st.host[0])
        if code != 0:
            _raise(code, st)
    if now - st.last_poll >= POLL_INTERVAL_S:
        idx = st.word.device.index
        if idx == torch.cuda.current_device():
            st.host.copy_(st.word, non_blocking=True)
            st.event.record()
        else:
            with torch.cuda.device(idx):
                st.host.copy_(st.word, non_blocking=True)
                st.event.record()
        st.pending = True
        st.last_poll = now
    return st.word


def check_device_status(device=None) -> None:
    """Synchronises and raises if any kernel launched so far on ``device`` gave up on a bounded
    device-side wait (the kernels never spin forever; they record a code and exit instead)."""
    st = _state(device)
    code = int(st.word.item())
    st.pending = False
    if code != 0:
        _raise(code, st)
