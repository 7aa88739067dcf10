"""What happens when a device-side wait runs out, exercised without hanging or faulting anything:
`b200attn_wait_timeout_selftest` runs the kernels' own bounded wait (`bounded_wait`) with a short limit on
a barrier that nothing arrives at, and follows the same give-up protocol (status code, abort flag for the
CTA's other warps, TMEM released, normal return)."""
import time

import pytest
import torch

from flagattention_b200 import _lib, flash_attention, status
from gpu_util import attention_forward, device, max_abs_diff

pytestmark = pytest.mark.gpu


def _run_selftest(limit_us, code, status_word):
    lib = _lib.load()
    out = torch.zeros(3, dtype=torch.int64, device=device())
    _lib.check(lib.b200attn_wait_timeout_selftest(limit_us, code, status_word.data_ptr(), out.data_ptr(),
                                                  torch.cuda.current_stream().cuda_stream), "wait_timeout_selftest")
    torch.cuda.synchronize()
    return out.tolist()


@pytest.mark.parametrize("limit_us,code", [(200, 1), (1000, 3)])
def test_wait_gives_up_records_its_code_and_the_context_stays_usable(limit_us, code):
    word = torch.zeros(1, dtype=torch.int32, device=device())
    gave_up, released, waited_ns = _run_selftest(limit_us, code, word)
    assert gave_up == 1
    assert released == 3, "the abort flag must release the CTA's other warps long before their own limit"
    assert limit_us * 1000 <= waited_ns <= limit_us * 1000 + 2_000_000
    assert word.item() == code
    # a second failure does not overwrite the first code
    _run_selftest(200, 4 if code != 4 else 2, word)
    assert word.item() == code
    # the context is intact and TMEM was released: a real kernel runs and is right
    q, k, v = (torch.randn(1, 2, 256, 64, device=device(), dtype=torch.float16) for _ in range(3))
    o = flash_attention(q, k, v)
    o_ref = attention_forward(q, k, v, False, upcast=True)
    o_low = attention_forward(q, k, v, False, upcast=False)
    assert max_abs_diff(o, o_ref) <= 2 * max_abs_diff(o_low, o_ref) + 1e-5


def test_reported_failure_reaches_the_caller():
    """A code in the library's per-device status word makes `check_device_status` raise, and, without
    any synchronisation by the caller, one of the next operator calls (`status.poll`)."""
    dev = device()
    word = status.status_word(dev)
    status.check_device_status(dev)
    _run_selftest(200, 2, word)
    with pytest.raises(RuntimeError, match="wait timeout"):
        status.check_device_status(dev)
    status.check_device_status(dev)                      # the word was cleared by the raise

    _run_selftest(200, 1, word)
    q, k, v = (torch.randn(1, 2, 128, 64, device=dev, dtype=torch.float16) for _ in range(3))
    deadline = time.monotonic() + 5.0
    with pytest.raises(RuntimeError, match="wait timeout"):
        while time.monotonic() < deadline:
            flash_attention(q, k, v)                     # polls before it launches
            time.sleep(0.01)
    status.check_device_status(dev)
    # kernels launched while a code is set leave at their first slow wait: run one clean call to be sure
    o = flash_attention(q, k, v)
    torch.cuda.synchronize()
    status.check_device_status(dev)
    assert torch.isfinite(o).all()
