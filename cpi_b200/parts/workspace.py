"""Named device buffers that live across steps, so that a step allocates nothing once it is warm."""
from __future__ import annotations

import torch


class Workspace:
    def __init__(self, device):
        self.device = device
        self._buffers: dict = {}
        self.generation = 0        # grows whenever a buffer is (re)allocated: captured graphs then hold stale addresses
        # A block may leave the write-back of its last sublayer to whoever touches the residual next (the next
        # block fuses it with its first read): (streams x, y, write weights, mixing matrix) or None.  Whoever
        # reads the residual without knowing about it calls `settle()` first.
        self.pending_writeback = None
        # A block whose sublayers read the residual itself may leave a copy of it in the activation dtype for the next
        # block: (address, tokens, width, dtype) of the residual that the buffer "post_norm_h" mirrors, or None.
        # `settle()` forgets it, so anything else that touches the residual in between invalidates the copy.
        self.residual_copy = None

    def settle(self) -> None:
        """Applies a write-back that a block has left pending (see `pending_writeback`)."""
        self.residual_copy = None
        p, self.pending_writeback = self.pending_writeback, None
        if p is not None:
            from ..csrc import lib as K
            K.hc_step(p[0], y=p[1], write=p[2], mix=p[3])

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < n:
            cap = max(n, 1)
            if buf is not None:
                cap = max(cap, int(buf.numel() * 1.5))
            buf = torch.empty(cap, dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self.generation += 1
        return buf[:n].view(*shape)

