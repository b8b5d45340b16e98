"""Three-phase (stable -> decay -> sft) CPU run used by the crash-restart test; optionally dies mid-phase with SIGKILL."""
import os
import signal
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import forge_train_harness_b200 as fth  # noqa: E402
from forge_train_harness_b200 import engine, train  # noqa: E402
from tests.test_parallel_cpu import base_cfg  # noqa: E402


def main():
    root, kill_at = sys.argv[1], int(sys.argv[2])
    cfg = base_cfg(steps=1)
    recipe = {"save_root": root, "order": ["stable", "decay", "sft"],
              "phases": {"stable": {"num_steps": 4, "save_interval": 2, "lr": 2e-3, "lr_schedule": "constant"},
                         "decay": {"num_steps": 4, "save_interval": 2, "lr": 2e-3, "min_lr": 2e-4, "lr_schedule": "wsd",
                                   "lr_decay_iters": 8, "lr_wsd_decay_iters": 4},
                         "sft": {"num_steps": 4, "save_interval": 2, "lr": 5e-4, "lr_schedule": "constant",
                                 "init_weights_only": True}}}
    if kill_at > 0:
        orig = fth.Trainer.train_step

        def step(self):
            r = orig(self)
            if self.step == kill_at and not os.path.exists(os.path.join(root, f"killed_{kill_at}")):
                open(os.path.join(root, f"killed_{kill_at}"), "w").close()
                sys.stdout.flush()
                os.kill(os.getpid(), signal.SIGKILL)  # host-side fault injection: the process dies between steps
            return r
        fth.Trainer.train_step = step
        engine.Trainer.train_step = step
    train.run_phases(cfg, recipe)


if __name__ == "__main__":
    main()
