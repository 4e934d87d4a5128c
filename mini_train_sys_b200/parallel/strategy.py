"""Strategy contract between the training scripts and a parallel layout.

``setup`` creates the process group, ``wrap_model`` returns what the trainer should
drive, ``barrier``/``teardown`` bracket the run (reference:
minitrain/distributed/strategy.py:6-36).  ``ProcessGroupMixin`` holds what every
multi-process strategy shares.
"""

from __future__ import annotations

import os
from datetime import timedelta
from typing import Protocol

import torch
import torch.distributed as dist


class ParallelStrategy(Protocol):
    name: str

    @property
    def rank(self) -> int: ...

    @property
    def world_size(self) -> int: ...

    def setup(self) -> None: ...

    def wrap_model(self, model: torch.nn.Module) -> torch.nn.Module: ...

    def barrier(self) -> None: ...

    def teardown(self) -> None: ...


class ProcessGroupMixin:
    process_group_backend: str = "auto"
    timeout_minutes: int = 30
    require_cuda: bool = False

    @property
    def local_rank(self) -> int:
        return int(os.environ.get("LOCAL_RANK", "0"))

    @property
    def rank(self) -> int:
        return dist.get_rank() if dist.is_initialized() else int(os.environ.get("RANK", "0"))

    @property
    def world_size(self) -> int:
        return dist.get_world_size() if dist.is_initialized() else int(os.environ.get("WORLD_SIZE", "1"))

    def setup(self) -> None:
        cuda = torch.cuda.is_available()
        if self.require_cuda and not cuda:
            raise RuntimeError(f"{getattr(self, 'name', 'this')} strategy requires a CUDA accelerator")
        if cuda:
            torch.cuda.set_device(self.local_rank)
        if dist.is_initialized():
            return
        backend = self.process_group_backend
        if backend == "auto":
            backend = "nccl" if cuda else "gloo"
        kwargs = {}
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", self.local_rank)
        attempt = int(os.environ.get("TORCHELASTIC_RESTART_COUNT", "0") or 0)
        if attempt > 0 and os.environ.get("MASTER_ADDR") and os.environ.get("MASTER_PORT"):
            # Restarted by the launcher after a rank failed (torchrun --max-restarts).  The launcher's store outlives the
            # failed workers; with the stock env:// rendezvous the restarted Gloo ranks found the dead ranks' addresses there
            # ("connection refused" in connectFullMesh).  Keys of this attempt go under a prefix of their own instead.
            store = dist.PrefixStore(f"mts/attempt_{attempt}",
                                     dist.TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]),
                                                   int(os.environ["WORLD_SIZE"]), False, timedelta(minutes=self.timeout_minutes)))
            kwargs.update(store=store, rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
        dist.init_process_group(backend=backend, timeout=timedelta(minutes=self.timeout_minutes), **kwargs)

    def barrier(self) -> None:
        if dist.is_initialized():
            if dist.get_backend() == "nccl":
                dist.barrier(device_ids=[self.local_rank])
            else:
                dist.barrier()

    def teardown(self) -> None:
        if dist.is_initialized():
            dist.destroy_process_group()
