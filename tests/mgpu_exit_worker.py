"""Two or more GPU ranks train with the fused engine; the last rank leaves in an orderly way between steps.

The survivors learn of it on the host (store notice) before they launch their next step, so no kernel ever waits for the
missing rank.  NVLS is off for this run (plain peer loads / stores only) and nothing is in flight when the rank leaves.
"""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from mini_train_sys_b200.models import MiniTransformer, ModelConfig, get_ops_backend
    from mini_train_sys_b200.parallel.comm import PeerCollectives
    from mini_train_sys_b200.parallel.flat_engine import FlatDataParallel
    from mini_train_sys_b200.runtime.config import OptimizerConfig
    from mini_train_sys_b200.runtime.health import PeerLostError, RankHealth
    from mini_train_sys_b200.train.optim import build_optimizer
    from mini_train_sys_b200.train.trainer import Trainer

    cfg = ModelConfig(vocab_size=1000, seq_len=128, n_layers=2, n_heads=4, hidden_size=256, intermediate_size=512, tie_word_embeddings=True)
    torch.manual_seed(0)
    model = MiniTransformer(cfg, get_ops_backend("native"), activation_dtype=torch.bfloat16).to(dev)
    coll = PeerCollectives(dev, max_units=8, wait_timeout_ms=2000, use_multimem=False)
    eng = FlatDataParallel(model, mode="shard", collectives=coll)
    tr = Trainer(eng, build_optimizer(eng, cfg=OptimizerConfig(lr=1e-3)), dev, use_fused_loss=True, precision="bf16", grad_clip_norm=1.0)
    health = RankHealth()
    g = torch.Generator().manual_seed(7 + rank)
    leaver = world - 1
    try:
        for step in range(5):
            health.check(max_age_seconds=30)
            t = torch.randint(0, 1000, (4, 129), generator=g)
            tr.train_step({"input_ids": t[:, :-1], "targets": t[:, 1:]})
            torch.cuda.synchronize(dev)                 # this rank has nothing in flight
            health.beat(step)
            if step == 1:
                dist.barrier()                          # everyone finished step 1: the leaver may go
                if rank == leaver:
                    health.leave("drained by the test")
                    print(f"LEFT rank={rank}", flush=True)
                    os._exit(0)
                import time
                time.sleep(1.0)                         # the notice is in the store before the survivors look
    except PeerLostError as exc:
        coll.check_status()                             # no device-side wait was started, so no timeout was recorded
        print(f"PASS survivor rank={rank} stopped on the host at step {step}: {exc}", flush=True)
        os._exit(0)
    print(f"FAIL rank={rank} finished all steps without noticing", flush=True)
    os._exit(1)


if __name__ == "__main__":
    main()
