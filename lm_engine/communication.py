"""Object broadcast helper (parity: lm_engine/communication.py:13-23)."""

from __future__ import annotations

import torch.distributed as dist


class Communication:
    @staticmethod
    def broadcast_object(obj, src: int, group: dist.ProcessGroup | None = None):
        """Broadcast a picklable object from global rank ``src`` to every member of ``group``."""
        holder = [obj]
        dist.broadcast_object_list(holder, src=src, group=group)
        return holder[0]
