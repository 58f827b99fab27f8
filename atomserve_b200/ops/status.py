"""The device's status words: how a kernel tells the host that it could not finish its work.

Kernels here never trap and never spin without end. A wait in a tcgen05 kernel that runs out of
polls writes which role gave up into word 0 and lets its block wind down (tensor memory freed,
output incomplete); the embedding gather writes 1 into word 1 when it meets a token id outside
the table. There is one set of words per device. The serving path copies them to pinned host
memory behind each step's kernels (`send_to_host`, no wait of its own) and looks at the copy once
the step's read of the sampled ids has returned (`problem_on_host`); tests and tools read the
device directly (`problem`).
"""

from __future__ import annotations

import torch

PIPELINE, EMBEDDING = 0, 1
_ROLES = {
    1: "GEMM: operand loads", 2: "GEMM: MMA issue", 3: "GEMM: epilogue", 4: "GEMM: accumulator hand-back",
}  # fmt: skip


def describe(words: list[int]) -> str | None:
    parts = []
    if words[PIPELINE]:
        code = words[PIPELINE]
        who = _ROLES.get(code, f"prefill attention, wait {code}" if 10 <= code <= 29 else ("the self-test" if code == 90 else f"wait {code}"))
        parts.append(f"a tcgen05 kernel gave up a bounded wait ({who}); its output is incomplete")
    if words[EMBEDDING]:
        parts.append("the embedding met a token id outside the vocabulary")
    return "; ".join(parts) or None


class DeviceStatus:
    WORDS = 4

    def __init__(self, device: torch.device):
        self.device = device
        self.words = torch.zeros(self.WORDS, dtype=torch.int32, device=device)
        self.pipeline, self.embedding = self.words[PIPELINE : PIPELINE + 1], self.words[EMBEDDING : EMBEDDING + 1]
        self._host = torch.zeros(self.WORDS, dtype=torch.int32, pin_memory=device.type == "cuda")
        self._seen = self._host.numpy()

    def send_to_host(self) -> None:
        """Queue a copy of the words to the host on the current stream, behind what was launched."""
        self._host.copy_(self.words, non_blocking=True)

    def problem_on_host(self) -> str | None:
        """What the last `send_to_host` brought, once the stream has been waited on (reading the
        step's result does that); clears the words after a report."""
        seen = self._seen
        if not (seen[PIPELINE] or seen[EMBEDDING]):
            return None
        text = describe(seen.tolist())
        self.words.zero_()
        self._host.zero_()
        return text

    def problem(self) -> str | None:
        """Read the device now (a synchronisation); clears the words after a report."""
        words = self.words.tolist()
        text = describe(words)
        if text:
            self.words.zero_()
        return text


def bounded_wait_selftest(device: torch.device | str = "cuda", polls: int = 4096) -> str | None:
    """Run the kernel that makes a bounded wait run out on purpose (csrc/wait_selftest.cu): it
    waits `polls` polls on a barrier that nothing arrives at, reports through the device's status
    word, frees its tensor memory and returns. Gives back the report that the status words then
    hold (and clears it), or raises if the block did not come back the expected way."""
    import ctypes

    from atomserve_b200.ops.library import KernelLibraryError, check, lib, ptr, stream

    status = status_for(device)
    fn = lib().asb_bounded_wait_selftest
    fn.argtypes, fn.restype = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p], ctypes.c_int
    freed = torch.zeros(1, dtype=torch.int32, device=status.device)
    check(fn(ptr(status.pipeline), polls, ptr(freed), stream()))
    outcome = int(freed.item())
    report = status.problem()
    if outcome != 1:
        raise KernelLibraryError(f"bounded-wait self-test: the block ended with outcome {outcome} (1 expected), report {report!r}")
    return report


_BY_DEVICE: dict[torch.device, DeviceStatus] = {}


def status_for(device: torch.device | str) -> DeviceStatus:
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    found = _BY_DEVICE.get(device)
    if found is None:
        found = _BY_DEVICE[device] = DeviceStatus(device)
    return found
