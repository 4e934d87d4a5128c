import random

import torch


def seed_everything(seed: int) -> None:
    """Seed python, torch CPU and every CUDA generator."""

    random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
