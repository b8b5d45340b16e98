"""gloo multi-rank parity: DP + ZeRO-1, TP (+SP, KV replication), PP (1F1B, interleaved), all vs one process."""
import pytest
import torch

import forge_train_harness_b200 as fth
from tests._mp import run_ranks


def base_cfg(steps=3, mbs=2, gbs=4, **par):
    model = fth.preset("tiny")
    import dataclasses
    model = dataclasses.replace(model, seq_length=32, padded_vocab_size=512, num_layers=4, hidden_size=64,
                                ffn_hidden_size=128, num_attention_heads=4, num_query_groups=2, head_dim=16,
                                mup_base_hidden_size=32)
    return fth.RunConfig(model=model, optim=fth.OptimConfig(lr=2e-3, lr_schedule="constant"),
                         parallel=fth.ParallelConfig(**par),
                         train=fth.TrainConfig(num_steps=steps, micro_batch_size=mbs, global_batch_size=gbs, seed=3,
                                               dtype="fp32", cuda_graph=False),
                         data=fth.DataConfig(prefetch_size=0))


def _train(rank, world, cfg):
    tr = fth.Trainer(cfg, device="cpu", quiet=True)
    out = []
    for _ in range(cfg.train.num_steps):
        r = tr.train_step()
        out.append((float(r["loss"]), float(r["grad_norm"])))
    tr.close()
    return out


def single(cfg):
    tr = fth.Trainer(cfg.replace(parallel={"tensor_parallel_size": 1, "pipeline_parallel_size": 1,
                                           "virtual_pipeline_stages": 1, "sequence_parallel": False,
                                           "use_distributed_optimizer": False}), device="cpu", quiet=True)
    out = []
    for _ in range(cfg.train.num_steps):
        r = tr.train_step()
        out.append((float(r["loss"]), float(r["grad_norm"])))
    tr.close()
    return out


def check(ref, got, tol=2e-4):
    for (l0, g0), (l1, g1) in zip(ref, got):
        assert abs(l0 - l1) / abs(l0) < tol, (ref, got)
        assert abs(g0 - g1) / abs(g0) < 10 * tol, (ref, got)


@pytest.mark.parametrize("zero", [False, True])
def test_dp2(zero):
    cfg = base_cfg(use_distributed_optimizer=zero, ddp_bucket_elems=20000)
    res = run_ranks(2, _train, cfg)
    check(single(cfg), res[0])
    assert res[0] == res[1]


@pytest.mark.parametrize("sp", [False, True])
def test_tp2(sp):
    cfg = base_cfg(tensor_parallel_size=2, sequence_parallel=sp)
    res = run_ranks(2, _train, cfg)
    check(single(cfg), res[0])


def _train_qk(rank, world, cfg):
    tr = fth.Trainer(cfg, device="cpu", quiet=True)
    out = []
    for _ in range(cfg.train.num_steps):
        r = tr.train_step()
        out.append((float(r["loss"]), float(r["grad_norm"])))
    w = torch.cat([tr.store.p(n).float().reshape(-1) for n in tr.store.params if n.endswith(("q_norm.weight", "k_norm.weight"))])
    tr.close()
    return out, w


@pytest.mark.parametrize("sp", [False, True])
def test_tp2_qk_norm_weights_stay_replicated(sp):
    """The per-head q / k norm weights see only the local heads under TP: their gradients are summed over the TP group
    with and without sequence parallelism, so every rank applies the same update and the run matches one process."""
    import dataclasses
    cfg = base_cfg(steps=4, tensor_parallel_size=2, sequence_parallel=sp)
    cfg = dataclasses.replace(cfg, model=dataclasses.replace(cfg.model, qk_norm=True),
                              optim=dataclasses.replace(cfg.optim, lr=2e-2))
    res = run_ranks(2, _train_qk, cfg)
    check(single(cfg), res[0][0])
    assert torch.equal(res[0][1], res[1][1])
    assert (res[0][1] - 1.0).abs().max() > 1e-3  # the norm weights did move


def _mtp_cfg(**par):
    import dataclasses
    cfg = base_cfg(steps=3, **par)
    return dataclasses.replace(cfg, model=dataclasses.replace(cfg.model, tie_embeddings=False, mtp_num_layers=1, mtp_loss_weight=0.3))


@pytest.mark.parametrize("sp", [False, True])
def test_tp2_with_mtp_branch(sp):
    """The Eagle / MTP branch under tensor (and sequence) parallelism: same losses as one process."""
    cfg = _mtp_cfg(tensor_parallel_size=2, sequence_parallel=sp)
    res = run_ranks(2, _train, cfg)
    check(single(cfg), res[0])


def test_pp2_with_mtp_branch_on_the_last_stage():
    """Pipeline parallelism with MTP: the last stage holds its own copy of the (untied) embedding for the branch's input
    tokens, and the two copies' gradients are summed, so the run matches one process."""
    cfg = _mtp_cfg(pipeline_parallel_size=2, gbs=8)
    res = run_ranks(2, _train, cfg)
    check(single(cfg), res[0])


@pytest.mark.parametrize("n", [1, 3, -1])
def test_last_n_layers_recompute_is_exact(n):
    """Layers whose activations are dropped and rebuilt in the backward pass give bitwise the same step."""
    cfg = base_cfg(steps=3)
    ref = single(cfg)
    got = single(cfg.replace(train={"recompute_num_layers": n}))
    assert ref == got


def test_tp4_kv_replication_sp():
    cfg = base_cfg(tensor_parallel_size=4, sequence_parallel=True)
    res = run_ranks(4, _train, cfg)
    check(single(cfg), res[0])


def test_pp2_1f1b():
    cfg = base_cfg(pipeline_parallel_size=2, gbs=8)
    res = run_ranks(2, _train, cfg)
    check(single(cfg), res[0])


def test_pp2_uneven_layer_split():
    """Three layers on the first stage, one (plus the head and the loss) on the last: same numbers as one process."""
    cfg = base_cfg(pipeline_parallel_size=2, pipeline_layer_split=(3, 1), gbs=8)
    res = run_ranks(2, _train, cfg)
    check(single(cfg.replace(parallel={"pipeline_layer_split": ()})), res[0])


def test_pp2_interleaved():
    cfg = base_cfg(pipeline_parallel_size=2, virtual_pipeline_stages=2, gbs=8)
    res = run_ranks(2, _train, cfg)
    check(single(cfg), res[0])


def test_tp2_pp2_dp2_sp_zero_interleaved():
    cfg = base_cfg(tensor_parallel_size=2, pipeline_parallel_size=2, virtual_pipeline_stages=2, sequence_parallel=True,
                   use_distributed_optimizer=True, gbs=16, ddp_bucket_elems=20000)
    res = run_ranks(8, _train, cfg)
    check(single(cfg), res[0])


def _train_overlap(rank, world, cfg):
    tr = fth.Trainer(cfg, device="cpu", quiet=True)
    out = []
    for _ in range(cfg.train.num_steps):
        r = tr.train_step()
        out.append((float(r["loss"]), float(r["grad_norm"])))
    n = getattr(tr.opt, "overlapped_buckets", 0)
    nb = len(tr.store.buckets)
    tr.close()
    return out, n, nb


@pytest.mark.parametrize("zero", [False, True])
def test_dp2_bucket_overlap_is_the_same_reduction(zero):
    """Buckets handed to the DP reduction while the last micro-batch's backward still runs give the same numbers as the
    reduction after the backward, and all buckets but the one holding the (tied) embedding go out early."""
    cfg = base_cfg(steps=3, mbs=2, gbs=8, use_distributed_optimizer=zero, ddp_bucket_elems=20000, overlap_grad_reduce=True)
    on = run_ranks(2, _train_overlap, cfg)
    off = run_ranks(2, _train_overlap, cfg.replace(parallel={"overlap_grad_reduce": False}))
    assert on[0][0] == off[0][0] and on[0][0] == on[1][0]
    assert off[0][1] == 0
    assert on[0][2] > 2 and 0 < on[0][1] < on[0][2]


def test_peer_memory_paths_are_for_groups_inside_one_node(monkeypatch):
    """TP inside a node and DP across nodes is the usual multi-node layout: the DP group then keeps the library collectives."""
    from forge_train_harness_b200.parallel import topology as T
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "8")
    assert not T.spans_nodes([0, 1, 2, 3]) and not T.spans_nodes(range(8)) and not T.spans_nodes([8, 9, 15])
    assert T.spans_nodes([0, 8]) and T.spans_nodes([3, 11, 19]) and T.spans_nodes(range(16))
    monkeypatch.delenv("LOCAL_WORLD_SIZE")
    monkeypatch.setenv("WORLD_SIZE", "4")      # a launcher that only states the world size: one node
    assert not T.spans_nodes([0, 1, 2, 3])
    monkeypatch.delenv("WORLD_SIZE")
    assert not T.spans_nodes([0])


def _device_init_sums(rank, world, cfg):
    tr = fth.Trainer(cfg, device="cpu", quiet=True, init_mode="device")
    out = (tr.topo.pp_rank, tr.topo.dp_rank, tr.topo.tp_rank,
           {k: (float(v.double().sum()), float(v.double().abs().sum())) for k, v in tr.store.params.items()})
    tr.close()
    return out


def test_device_init_is_keyed_by_parameter_name():
    """Per-shard initialisation: layers on different pipeline stages must not draw the same numbers (a position-keyed stream
    made layer k of stage 1 a copy of layer k of stage 0), while the tied embedding's two copies, DP replicas and
    TP-replicated tensors stay identical and TP shards differ."""
    cfg = base_cfg(tensor_parallel_size=2, pipeline_parallel_size=2, sequence_parallel=True, use_distributed_optimizer=True, gbs=16)
    res = run_ranks(8, _device_init_sums, cfg)
    by = {(pp, dp, tp): st for pp, dp, tp, st in res}
    s0, s1 = by[(0, 0, 0)], by[(1, 0, 0)]
    assert s0["tok_embeddings.weight"] == s1["tok_embeddings.weight"]                       # tied copies
    mats0 = sorted(v for k, v in s0.items() if k.endswith("wqkv.weight"))
    mats1 = sorted(v for k, v in s1.items() if k.endswith("wqkv.weight"))
    assert len(mats0) == 2 and len(mats1) == 2 and not set(mats0) & set(mats1)               # no layer duplicated across stages
    assert len({v for st in (s0, s1) for k, v in st.items() if k.endswith("w2.weight")}) == 4
    for pp in (0, 1):
        for tp in (0, 1):
            assert by[(pp, 0, tp)] == by[(pp, 1, tp)]                                        # DP replicas
        a, b = by[(pp, 0, 0)], by[(pp, 0, 1)]
        for k in a:
            if k.endswith("norm.weight"):
                assert a[k] == b[k]                                                          # TP-replicated
            else:
                assert a[k] != b[k], k                                                       # TP shards
