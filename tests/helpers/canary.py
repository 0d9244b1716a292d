"""Canary-padded buffers for kernel tests: a tensor is carved out of a larger allocation whose rows before and after
it hold a poison pattern; ``check`` fails when a kernel wrote outside the tensor it was given."""
import torch

POISON = 12288.0  # exactly representable in bf16


class Canary:
    def __init__(self, rows: int, cols: int, dtype=torch.bfloat16, device="cuda", guard: int = 16, fill=None):
        self.guard = guard
        self.buf = torch.full((rows + 2 * guard, cols), POISON, dtype=dtype, device=device)
        self.t = self.buf[guard:guard + rows]
        if fill is not None:
            self.t.copy_(fill)

    def check(self, what: str = "kernel"):
        g = self.guard
        before, after = self.buf[:g].float(), self.buf[-g:].float()
        assert bool((before == POISON).all()) and bool((after == POISON).all()), f"{what} wrote outside its output tensor"
