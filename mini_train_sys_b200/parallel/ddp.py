"""Data parallelism.

Two engines share the strategy name ``ddp``:

* ``nccl`` - ``torch.nn.parallel.DistributedDataParallel`` with the reference's knobs
  (minitrain/distributed/ddp.py:9-72; 25 MB buckets, gradients as bucket views).  It
  also serves CPU/gloo runs.  This is the measured baseline.
* ``fused`` - replicated parameters in one flat fp32 buffer; gradients are reduced by
  the own peer-memory all-reduce kernel which also applies the AdamW update to the
  slice this rank reduces (parallel/flat_engine.py).
"""

from __future__ import annotations

import torch
from torch.nn.parallel import DistributedDataParallel

from mini_train_sys_b200.parallel.strategy import ProcessGroupMixin


class DDPStrategy(ProcessGroupMixin):
    name = "ddp"

    def __init__(self, *, process_group_backend: str = "auto", timeout_minutes: int = 30,
                 broadcast_buffers: bool = False, bucket_cap_mb: int = 25, find_unused_parameters: bool = False,
                 gradient_as_bucket_view: bool = True, static_graph: bool = False, engine: str = "nccl",
                 comm=None) -> None:
        self.process_group_backend = process_group_backend
        self.timeout_minutes = timeout_minutes
        self.ddp_kwargs = dict(broadcast_buffers=broadcast_buffers, bucket_cap_mb=bucket_cap_mb,
                               find_unused_parameters=find_unused_parameters,
                               gradient_as_bucket_view=gradient_as_bucket_view, static_graph=static_graph)
        self.engine = engine
        self.comm = comm

    def resolved_engine(self) -> str:
        if self.engine == "auto":
            return "fused" if torch.cuda.is_available() else "nccl"
        return self.engine

    def wrap_model(self, model: torch.nn.Module) -> torch.nn.Module:
        if self.resolved_engine() == "fused":
            from mini_train_sys_b200.parallel.flat_engine import FlatDataParallel

            return FlatDataParallel(model, mode="replicate", comm=self.comm, bucket_cap_mb=self.ddp_kwargs["bucket_cap_mb"])
        kwargs = dict(self.ddp_kwargs)
        if torch.cuda.is_available():
            kwargs.update(device_ids=[self.local_rank], output_device=self.local_rank)
        return DistributedDataParallel(model, **kwargs)
