"""Child process of ``test_legacy_codec_round_trips_with_the_reference``: imports the UNMODIFIED reference engine
(installed under ``baseline/_ref``; it reads its geometry from the environment at import) and exchanges
``step_<N>/training_state.pt`` files with this package's legacy codec in both directions.  The CUDA generator calls of
the reference's codec are replaced by CPU stand-ins: there is no GPU where this runs."""
import os
import pickle
import random
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))


def main(tmp):
    import forge_train_harness_b200 as fth
    from forge_train_harness_b200.ckpt import manager as ckpt
    from tests.test_parallel_cpu import base_cfg
    from training_engine_tensor import train_loop as ref  # noqa: E402  (needs the geometry variables)
    cuda_state = {}
    torch.cuda.get_rng_state = lambda *a, **k: torch.arange(16, dtype=torch.uint8)
    torch.cuda.set_rng_state = lambda s, *a, **k: cuda_state.update(v=s.clone())

    cfg = base_cfg(steps=2).replace(ckpt={"format": "legacy"})
    tr = fth.Trainer(cfg, device="cpu", quiet=True)
    tr.train_step()
    tr.train_step()
    np.random.seed(123)
    random.seed(321)
    want_np, want_py = np.random.get_state(), random.getstate()
    ours = os.path.join(tmp, "ours")
    ckpt.save(tr, ours)

    # (1) a file written here, read by the reference's load_checkpoint
    names = [s.name for s in tr.store.specs]
    masters = [torch.zeros(tr.store.shapes[n]) for n in names]
    m = {p.data_ptr(): torch.zeros_like(p) for p in masters}
    v = {p.data_ptr(): torch.zeros_like(p) for p in masters}
    st = {p.data_ptr(): torch.zeros(()) for p in masters}
    np.random.seed(0)
    random.seed(0)
    step = ref.load_checkpoint(ours, masters, m, v, st, rank=0)
    assert step == 2, step
    full = tr.opt.gather_full_state()
    for n, p in zip(names, masters):
        o, cnt = tr.store.offsets[n]
        assert torch.equal(p.reshape(-1), full["master"][o:o + cnt]), n
        assert torch.equal(m[p.data_ptr()].reshape(-1), full["exp_avg"][o:o + cnt]), n
        assert torch.equal(v[p.data_ptr()].reshape(-1), full["exp_avg_sq"][o:o + cnt]), n
        assert float(st[p.data_ptr()]) == 2.0
    got_np = np.random.get_state()
    assert got_np[0] == want_np[0] and np.array_equal(got_np[1], want_np[1]) and got_np[2:] == want_np[2:]
    assert random.getstate() == want_py
    assert cuda_state["v"].numel() == 16

    # (2) a file written by the reference's save_checkpoint, read here
    for p in masters:
        p.add_(0.25)
    np.random.seed(77)
    random.seed(78)
    torch.manual_seed(79)
    want = (np.random.get_state(), random.getstate(), torch.get_rng_state())
    theirs = os.path.join(tmp, "theirs")
    ref.save_checkpoint(theirs, 5, masters, m, v, {k: torch.tensor(5.0) for k in st}, rank=0)
    np.random.seed(1)
    random.seed(1)
    torch.manual_seed(1)
    tr2 = fth.Trainer(cfg, device="cpu", quiet=True)
    assert ckpt.load(tr2, theirs) == 5 and tr2.opt.step_count == 5
    full2 = tr2.opt.gather_full_state()
    for n, p in zip(names, masters):
        o, cnt = tr2.store.offsets[n]
        assert torch.equal(full2["master"][o:o + cnt], p.reshape(-1)), n
        assert torch.equal(tr2.store.p(n), p), n
    got_np = np.random.get_state()
    assert np.array_equal(got_np[1], want[0][1]) and got_np[2:] == want[0][2:]
    assert random.getstate() == want[1] and torch.equal(torch.get_rng_state(), want[2])
    # a file of the older form of this codec (RNG bytes wrapped in uint8 tensors) still loads
    sd = torch.load(os.path.join(theirs, "step_5", "training_state.pt"), weights_only=True)
    sd["rng_numpy"] = torch.frombuffer(bytearray(sd["rng_numpy"]), dtype=torch.uint8)
    sd["rng_random"] = torch.frombuffer(bytearray(sd["rng_random"]), dtype=torch.uint8)
    old = os.path.join(tmp, "old", "step_5")
    os.makedirs(old)
    torch.save(sd, os.path.join(old, "training_state.pt"))
    assert ckpt.load(tr2, os.path.join(tmp, "old")) == 5
    tr.close()
    tr2.close()
    print("LEGACY_CODEC_OK")


if __name__ == "__main__":
    main(sys.argv[1])
