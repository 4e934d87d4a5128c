import torch


class SingleDeviceStrategy:
    """World of one: no process group; ``barrier`` drains the CUDA stream for timing."""

    name = "single"
    rank = 0
    world_size = 1

    def setup(self) -> None:
        pass

    def wrap_model(self, model: torch.nn.Module) -> torch.nn.Module:
        return model

    def barrier(self) -> None:
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def teardown(self) -> None:
        pass
