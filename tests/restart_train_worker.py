"""``scripts/train.py`` with one scripted crash, for the restart test (CPU, Gloo): rank 1 exits without a word right after
optimizer step ``CRASH_AFTER_STEP``, once (a marker file remembers that it happened).  Everything else is the stock entry
point, so what the test exercises is the launcher's restart and the entry point's ``--resume auto``."""

import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "scripts"))

import train as entry  # noqa: E402  (scripts/train.py)

from mini_train_sys_b200.train.trainer import Trainer  # noqa: E402

crash_after = int(os.environ["CRASH_AFTER_STEP"])
marker = Path(os.environ["CRASH_MARKER"])
original = Trainer.train_step


def train_step_with_one_crash(self, batch):
    loss = original(self, batch)
    if int(os.environ.get("RANK", "0")) == 1 and self.state.step == crash_after and not marker.exists():
        marker.write_text("crashed once\n")
        os._exit(17)
    return loss


Trainer.train_step = train_step_with_one_crash

if __name__ == "__main__":
    entry.main()
