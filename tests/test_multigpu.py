"""Multi-GPU parity on real devices: fused peer-memory DP path vs NCCL path vs one GPU; TP+SP and PP on NCCL."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(mode, nproc, env=None):
    e = dict(os.environ)
    e.update(env or {})
    e.setdefault("NCCL_NVLS_ENABLE", "0")
    cmd = [sys.executable, "-m", "forge_train_harness_b200.runtime.launcher", "--nproc", str(nproc), "--",
           sys.executable, os.path.join(ROOT, "tests", "_mgpu_worker.py"), mode]
    p = subprocess.run(cmd, cwd=ROOT, env=e, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    line = [ln for ln in p.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    return json.loads(line[7:])


def close(a, b, tol):
    """Relative loss deviation below ``tol`` at every step, grad-norm deviation below ``max(2 tol, 2 %)``."""
    for (l0, g0), (l1, g1) in zip(a["steps"], b["steps"]):
        assert abs(l0 - l1) / abs(l0) < tol, (a, b)
        assert abs(g0 - g1) / abs(g0) < max(2 * tol, 2e-2), (a, b)


needs2 = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")


@needs2
def test_fused_dp_bucket_pulls_overlap_the_backward_eager_and_in_the_graph():
    """The peer-memory reduce-scatter runs bucket by bucket behind the last micro-batch's backward (side stream, device-
    numbered flag barrier), eagerly and inside the captured graph; same numbers as pulling after the backward."""
    late = run("dp_zero_late", 2)
    eager = run("dp_zero", 2)
    graph = run("dp_zero:graph", 2)
    assert late["paths"]["dp_buckets_overlapped_with_backward"] == 0
    assert eager["paths"]["dp_buckets_overlapped_with_backward"] > 0 and eager["paths"]["dp_buckets"] > 2
    assert graph["paths"]["dp_buckets_overlapped_with_backward"] > 0 and graph["paths"]["cuda_graph"]
    close(late, eager, 1e-3)
    close(late, graph, 1e-3)


@needs2
def test_fused_dp_matches_nccl_and_single_gpu():
    single = run("single", 1)
    nccl = run("dp_zero", 2, {"FORGE_FUSED_DP": "0"})
    fused = run("dp_zero", 2, {"FORGE_FUSED_DP": "1"})
    assert fused["fused"] and not nccl["fused"]
    close(single, nccl, 5e-3)
    close(nccl, fused, 5e-3)


@needs2
def test_tp2_sp_fused_and_nccl_and_pp2_match_single_gpu():
    single = run("single", 1)
    nccl = run("tp_sp", 2, {"FORGE_FUSED_TP": "0"})
    fused = run("tp_sp", 2, {"FORGE_FUSED_TP": "1"})
    assert fused["fused"] and not nccl["fused"]
    close(single, nccl, 5e-3)
    close(single, fused, 5e-3)
    close(single, run("pp", 2), 5e-3)


@needs2
def test_tp2_layer_loops_replayed_from_cuda_graphs_match_eager():
    """After one eager step the layer loops run from CUDA graphs (fused TP kernels with device-numbered ordering inside):
    same losses as the eager run of the same layout, and the graphs really were replayed."""
    eager = run("tp_sp", 2)
    graph = run("tp_sp:graph", 2)
    assert graph["graph_replays"] > 0 and eager["graph_replays"] == 0 and graph["fused"]
    close(eager, graph, 5e-3)
    pp = run("pp:graph", 2)
    assert pp["graph_replays"] > 0
    close(run("single", 1), pp, 5e-3)


needs4 = pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")


@needs4
def test_tp4_with_replicated_kv_heads_fused_and_nccl_match_single_gpu():
    """2 KV heads on 4 tensor-parallel ranks: each KV head lives on two ranks and its weight gradient is summed over them."""
    single = run("single", 1)
    nccl = run("tp_sp", 4, {"FORGE_FUSED_TP": "0"})
    fused = run("tp_sp", 4, {"FORGE_FUSED_TP": "1"})
    assert fused["fused"] and not nccl["fused"]
    close(single, nccl, 5e-3)
    close(single, fused, 5e-3)


@needs4
def test_tp2_pp2_and_interleaved_match_single_gpu():
    single = run("single", 1)
    close(single, run("tp2pp2", 4), 5e-3)
    close(single, run("tp2pp2v2", 4), 5e-3)
    g = run("tp2pp2v2:graph", 4)
    assert g["graph_replays"] > 0
    close(single, g, 5e-3)


@needs4
def test_fused_dp_under_tp_and_under_pp_matches_single_gpu():
    """The peer-memory DP path with two data-parallel groups side by side (TP 2 x DP 2, PP 2 x DP 2), fused and NCCL."""
    single = run("single", 1)
    for mode in ("tp2dp2", "pp2dp2"):
        nccl = run(mode, 4, {"FORGE_FUSED_DP": "0", "FORGE_FUSED_TP": "0"})
        fused = run(mode, 4)
        assert fused["fused"]
        close(single, nccl, 5e-3)
        close(single, fused, 5e-3)


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")
def test_tp2_pp2_dp2_matches_single_gpu():
    close(run("single", 1), run("tp2pp2", 8), 5e-3)
