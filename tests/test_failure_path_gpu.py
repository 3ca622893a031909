"""The failure path, exercised without faulting anything: every device-side wait of the library is
bounded; a wait that runs out records a code in the per-device status word and the kernel ends
normally; ``forge_read_status`` turns the code into ``FORGE_ERR_TIMEOUT`` (``ForgeLibraryError`` in
Python) and clears the word, and the context stays usable for the next launch."""

import time

import pytest
import torch

from forge_b200 import _lib
from forge_b200 import kernel as K
from tests.util import ADAMW

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", torch.cuda.current_device())


def test_status_word_is_reported_and_cleared():
    dev = _dev()
    word = _lib.status_word(dev)
    assert _lib.read_status(dev) == 0
    word[0:1].fill_(104)                       # what a kernel that gave up on a state-ring wait would leave
    with pytest.raises(_lib.ForgeLibraryError, match="104") as ei:
        _lib.read_status(dev)
    assert f"code {_lib.FORGE_ERR_TIMEOUT}" in str(ei.value)
    assert word[0].item() == 0, "reading the status clears it"
    assert _lib.read_status(dev) == 0


def test_wait_that_nothing_satisfies_gives_up_and_reports():
    dev = _dev()
    lib = _lib.load()
    word = _lib.status_word(dev)
    stream = torch.cuda.current_stream().cuda_stream
    t0 = time.perf_counter()
    assert lib.forge_selftest_wait_timeout(word.data_ptr(), 50_000, stream) == 0      # 50 us limit
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0, "the kernel must end by itself, long before the 2 s production limit"
    assert word[0].item() == 190
    with pytest.raises(_lib.ForgeLibraryError, match="190"):
        _lib.read_status(dev)
    assert _lib.read_status(dev) == 0
    # argument checks of the entry itself
    assert lib.forge_selftest_wait_timeout(None, 50_000, stream) == _lib.FORGE_ERR_INVALID_ARG
    assert lib.forge_selftest_wait_timeout(word.data_ptr(), 0, stream) == _lib.FORGE_ERR_INVALID_ARG
    assert lib.forge_selftest_wait_timeout(word.data_ptr(), 2_000_000_000, stream) == _lib.FORGE_ERR_INVALID_ARG
    # the context is intact: a normal update runs and reports no error
    w = torch.zeros(128, 256, dtype=torch.bfloat16, device=dev)
    m, v = torch.zeros_like(w), torch.zeros_like(w)
    K.fused_grad_adamw(torch.ones(64, 128, dtype=torch.bfloat16, device=dev),
                       torch.ones(64, 256, dtype=torch.bfloat16, device=dev), w, m, v, **ADAMW)
    assert _lib.read_status(dev) == 0
    assert w.abs().sum().item() > 0


def test_first_error_wins_until_it_is_read():
    """Kernels record their code with a compare-and-swap against 0: a later failure does not hide the
    first one."""
    dev = _dev()
    lib = _lib.load()
    word = _lib.status_word(dev)
    word[0:1].fill_(106)
    assert lib.forge_selftest_wait_timeout(word.data_ptr(), 20_000, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert word[0].item() == 106
    with pytest.raises(_lib.ForgeLibraryError, match="106"):
        _lib.read_status(dev)
