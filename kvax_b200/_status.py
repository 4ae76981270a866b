"""The device status word of the attention kernels, kept where the host can read it at any time.

Every barrier wait inside the kernels is bounded; a wait that gives up writes 100 + barrier id
to a status word and the kernel runs to its end (nothing traps).  The word lives in page-locked
host memory that the device addresses directly: the kernels only touch it on failure, and the
host can look at it without synchronising a stream.  One word per device, shared by every call.
"""
from __future__ import annotations

import ctypes as C

import torch

from kvax_b200 import _lib

_words: dict[int, tuple[torch.Tensor, int]] = {}


def status_word(device: torch.device) -> tuple[torch.Tensor, int]:
    """(pinned host int32[1], address of that word as the device sees it)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    entry = _words.get(idx)
    if entry is None:
        word = torch.zeros(1, dtype=torch.int32).pin_memory()
        dev_ptr = C.c_void_p()
        with torch.cuda.device(idx):
            rc = _lib.load().kvax_b200_host_word_device_pointer(word.data_ptr(), C.byref(dev_ptr))
        _lib.check(rc, "kvax_b200_host_word_device_pointer")
        entry = (word, int(dev_ptr.value))
        _words[idx] = entry
    return entry


def last_status(device: torch.device | None = None) -> int:
    """Status code of the device (0 = ok) as of the kernels that have finished so far."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return int(status_word(device)[0][0])


def check_last_status(device: torch.device | None = None, synchronize: bool = False) -> None:
    """Raises KvaxB200Error when a kernel on `device` reported a failure, and clears the word.
    Without `synchronize` only kernels that have already finished are covered."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    if synchronize:
        torch.cuda.synchronize(device)
    word, _ = status_word(device)
    code = int(word[0])
    if code != 0:
        word[0] = 0
        what = "the shared memory window was misaligned" if code == 90 else "a bounded wait gave up (100 + barrier id)"
        raise _lib.KvaxB200Error(f"attention kernel on {device} reported status {code}: {what}; "
                                 "outputs of that call are not valid")
