import torch


class SingleDeviceStrategy:
    """World of one: no process group; ``barrier`` drains the CUDA stream for timing.

    With ``engine="fused"`` the model is still wrapped by the flat engine (fp32 master weights, bf16
    replicas, device-side clipping fused into AdamW), which is the single-rank case of the sharded
    strategies; with ``engine="nccl"`` the model is returned untouched, as in the reference
    (minitrain/distributed/single.py:4-21).
    """

    name = "single"
    rank = 0
    world_size = 1

    def __init__(self, *, engine: str = "nccl", comm=None) -> None:
        self.engine = engine
        self.comm = comm

    def resolved_engine(self) -> str:
        return self.engine

    def setup(self) -> None:
        pass

    def wrap_model(self, model: torch.nn.Module) -> torch.nn.Module:
        if self.engine == "fused":
            from mini_train_sys_b200.parallel.flat_engine import FlatDataParallel

            return FlatDataParallel(model, mode="shard", comm=self.comm)
        return model

    def barrier(self) -> None:
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def teardown(self) -> None:
        pass
