"""Point-to-point messages between ranks: the send / receive pair that pipeline stages need.

The reference has no pipeline parallelism; its message-passing examples
(examples/06_message_passing/message_passing_put.py:17-81, examples/31_message_passing/example.py)
show the primitive: ``put`` the payload into the peer's heap, then set a flag there with release
semantics; the consumer spins on the flag with acquire semantics. ``P2PChannel`` is that protocol
as an object, driven from the host with the one-sided operations of ``ctx.rma`` (stream-ordered
kernels on a GPU, plain memory operations on the CPU backend):

* every rank owns, for every possible sender, ``depth`` mailbox slots and a ``full`` word per slot;
  message ``n`` of a sender goes to slot ``(n - 1) % depth`` and sets ``full`` to ``n``;
* the receiver waits for ``full >= n`` (bounded), copies the payload out and writes ``n`` into the
  sender's ``ack`` word for that slot; a sender about to reuse a slot first waits for the
  acknowledgement of the message that used it before (back-pressure instead of overwriting).

Sequence numbers instead of 0 / 1 flags mean nothing is ever reset, so there is no window in which a
late reader sees a cleared flag. Every wait has a limit and raises ``TimeoutError``; the context
stays usable.
"""
from __future__ import annotations

import torch


class P2PChannel:
    """Mailboxes for ``shape`` / ``dtype`` messages between any two ranks of the context, ``depth`` slots
    per sender (collective constructor; see the module docstring for the protocol)."""

    def __init__(self, ctx, shape, dtype=torch.float32, depth: int = 2, timeout_ms: int = 5000):
        if depth < 1:
            raise ValueError("depth must be at least 1")
        self.ctx, self.shape, self.dtype, self.depth, self.timeout_ms = ctx, tuple(shape), dtype, depth, timeout_ms
        W = ctx.get_num_ranks()
        # all three live at the same offsets on every rank (collective allocation)
        self.slots = ctx.zeros((W, depth) + self.shape, dtype=dtype)       # [sender, slot]: in the receiver's heap
        self.full = ctx.zeros((W, depth), dtype=torch.int32)               # [sender, slot]: number of the message held
        self.ack = ctx.zeros((W, depth), dtype=torch.int32)                # [receiver, slot]: in the sender's heap
        self._sent = [0] * W
        self._received = [0] * W
        ctx.barrier()

    def send(self, tensor: torch.Tensor, to_rank: int) -> int:
        """Deliver ``tensor`` into ``to_rank``'s mailbox; returns the message number. Blocks (bounded)
        only when ``depth`` earlier messages to that rank are still unacknowledged."""
        ctx, me = self.ctx, self.ctx.get_rank()
        if to_rank == me or not 0 <= to_rank < ctx.get_num_ranks():
            raise ValueError(f"cannot send to rank {to_rank}")
        if tuple(tensor.shape) != self.shape or tensor.dtype != self.dtype:
            raise ValueError(f"this channel carries {self.dtype} tensors of shape {self.shape}")
        n = self._sent[to_rank] + 1
        i = (n - 1) % self.depth
        if n > self.depth and not ctx.wait_flag(self.ack[to_rank, i:i + 1], n - self.depth, self.timeout_ms):
            raise TimeoutError(f"rank {to_rank} has not taken message {n - self.depth} from rank {me} within {self.timeout_ms} ms")
        ctx.rma.put(tensor.contiguous(), self.slots[me, i], to_rank=to_rank)
        # the payload is ordered before the flag: release at system scope, after the put on the same stream
        ctx.rma.atomic_xchg(self.full[me, i:i + 1], n, to_rank=to_rank, sem="release", scope="sys")
        self._sent[to_rank] = n
        return n

    def recv(self, from_rank: int, out: torch.Tensor | None = None) -> torch.Tensor:
        """The next message of ``from_rank`` (a copy, or ``out`` filled); raises ``TimeoutError`` if it
        does not arrive within the channel's limit."""
        ctx, me = self.ctx, self.ctx.get_rank()
        if from_rank == me or not 0 <= from_rank < ctx.get_num_ranks():
            raise ValueError(f"cannot receive from rank {from_rank}")
        n = self._received[from_rank] + 1
        i = (n - 1) % self.depth
        if not ctx.wait_flag(self.full[from_rank, i:i + 1], n, self.timeout_ms):
            raise TimeoutError(f"message {n} from rank {from_rank} has not reached rank {me} within {self.timeout_ms} ms")
        payload = self.slots[from_rank, i]
        if out is None:
            out = payload.clone()
        else:
            out.copy_(payload)
        # tell the sender that the slot is free again (its ack word for me, in its heap)
        ctx.rma.atomic_xchg(self.ack[me, i:i + 1], n, to_rank=from_rank, sem="release", scope="sys")
        self._received[from_rank] = n
        return out

    def pending(self, from_rank: int) -> bool:
        """True when the next message of ``from_rank`` has already arrived (no waiting)."""
        n = self._received[from_rank] + 1
        return int(self.full[from_rank, (n - 1) % self.depth].item()) >= n
