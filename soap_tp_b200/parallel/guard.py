"""Debug-mode guard against ranks that disagree about the collective they are entering.

Every public op of this package is collective: all ranks of the grid must call the same op, for the same
parameter, with the same layout arguments, in the same order.  A rank that calls with another ``global_shape``
or skips a parameter does not fail by itself -- it reads the wrong panels or waits for a peer that never comes.
The reference relies on MPI and ``torch.distributed`` pairing up whatever is called
(``src/soap_tp/ops/factorizations.py:85-101``) and only checks the permutation vectors
(``src/soap_tp/ops/optimizer.py:439-452``).  With ``SOAP_TP_CHECK_COLLECTIVES=1`` every op first exchanges a
description of the call over the control plane and raises :class:`SoapCollectiveMismatch` on EVERY rank if
the descriptions differ, before anything touches the data plane.  Off by default: it costs one small host-side
all-gather per op.
"""
from __future__ import annotations

import os
from typing import Any, List, Optional

import torch.distributed as dist


class SoapCollectiveMismatch(RuntimeError):
    """Ranks entered different collectives, or the same one with different arguments."""


def enabled() -> bool:
    return os.environ.get("SOAP_TP_CHECK_COLLECTIVES", "0") == "1"


def _normalise(value: Any) -> Any:
    if isinstance(value, (list, tuple)):
        return tuple(_normalise(v) for v in value)
    if isinstance(value, float):
        return repr(value)
    return value


def check_collective(op: str, *fields: Any, group=None) -> None:
    """All ranks of ``group`` must be entering ``op`` with equal ``fields`` (no-op unless enabled)."""
    if not enabled() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    mine = (op,) + tuple(_normalise(f) for f in fields)
    everyone: List[Optional[tuple]] = [None] * dist.get_world_size(group)
    dist.all_gather_object(everyone, mine, group=group)
    if any(entry != everyone[0] for entry in everyone):
        lines = "\n".join(f"  rank {rank}: {entry}" for rank, entry in enumerate(everyone))
        raise SoapCollectiveMismatch(f"ranks disagree about the collective they are entering:\n{lines}")
