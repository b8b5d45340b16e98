"""Environment verification: is this box able to build and run the engine?

    python -m forge_train_harness_b200.harness env

Checks the pins this tree was built and measured against (interpreter, torch, CUDA toolkit with an sm_100a capable nvcc,
NCCL through torch), that the in-tree extension is built and loads, that its kernels were compiled for the GPU that is
present, and that a GPU (if any) is a compute-capability-10.0 part.  Every check yields ``(name, ok, detail)``; nothing here
changes a setting of the machine.  Counterpart of the reference's environment scripts, which parse their pins out of a
Dockerfile and verify torch / CUDA / flash-attn / triton versions before a gate sweep (env/_pins.py:47-66,
env/verify_env_torch.sh); this engine needs neither flash-attn nor triton.
"""
from __future__ import annotations

import os
import re
import shutil
import subprocess
import sys

PINS = {"python": (3, 10), "torch": (2, 6), "cuda_toolkit": (12, 8)}


def _ver(text: str) -> tuple[int, ...]:
    return tuple(int(x) for x in re.findall(r"\d+", text)[:3])


def checks(nvcc_output: str | None = None) -> list[tuple[str, bool, str]]:
    out = []
    out.append(("python", sys.version_info[:2] >= PINS["python"], sys.version.split()[0]))
    try:
        import torch
        tv = _ver(torch.__version__)
        out.append(("torch", tv[:2] >= PINS["torch"], torch.__version__))
        import torch.distributed as dist
        out.append(("torch.distributed backends", dist.is_available() and dist.is_gloo_available(),
                    f"gloo={dist.is_gloo_available()} nccl={dist.is_nccl_available()}"))
        has_gpu = torch.cuda.is_available()
        if has_gpu:
            cap = torch.cuda.get_device_capability(0)
            out.append(("gpu compute capability", cap == (10, 0), f"{torch.cuda.get_device_name(0)} sm_{cap[0]}{cap[1]}"))
        else:
            out.append(("gpu compute capability", True, "no GPU visible (build / CPU tests only)"))
    except Exception as e:  # noqa: BLE001
        out.append(("torch", False, f"{type(e).__name__}: {e}"))
        has_gpu = False
    if nvcc_output is None:
        nvcc = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
        try:
            nvcc_output = subprocess.run([nvcc, "--version"], capture_output=True, text=True, timeout=30).stdout
        except Exception as e:  # noqa: BLE001
            nvcc_output = f"unavailable: {e}"
    m = re.search(r"release (\d+)\.(\d+)", nvcc_output)
    out.append(("cuda toolkit (nvcc, sm_100a)", bool(m) and (int(m.group(1)), int(m.group(2))) >= PINS["cuda_toolkit"],
                m.group(0) if m else nvcc_output.strip()[:80]))
    so = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_C.so")
    built = os.path.isfile(so)
    out.append(("extension built in-tree", built, so if built else "run python -m forge_train_harness_b200.csrc.build"))
    if built and has_gpu:
        try:
            from ..ops import cuda_ops  # noqa: F401
            out.append(("extension loads", True, "forge_train_harness_b200._C"))
        except Exception as e:  # noqa: BLE001
            out.append(("extension loads", False, f"{type(e).__name__}: {e}"))
    return out


def main(argv=None) -> int:
    rows = checks()
    width = max(len(r[0]) for r in rows)
    for name, ok, detail in rows:
        print(f"{'ok  ' if ok else 'FAIL'} {name.ljust(width)}  {detail}")
    return 0 if all(r[1] for r in rows) else 1


if __name__ == "__main__":
    sys.exit(main())
