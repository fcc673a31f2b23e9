"""CPU test of the expert-parallel exchange protocol: two gloo ranks run
ExpertParallelEngine over a numpy implementation of the device stages; the gathered result
must equal the single-process oracle bit for bit."""
import importlib
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import __graft_entry__ as entry


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, tokens, result_dir, capacity):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        entry.load_package()
        synthetic = importlib.import_module("nemotron_inference_b200.synthetic")
        ep = importlib.import_module("nemotron_inference_b200.expert_parallel")
        import helpers
        from ep_cpu_stages import NumpyStages
        cfg = synthetic.baseline_config(64, experts=32, hidden=128, routed=64, shared=128, top_k=4)
        data = synthetic.make_layer(cfg, seed=17, device="cpu", norm_weight_uniform=True)
        ocfg, ow = helpers.oracle_config(cfg), helpers.oracle_weights(data)
        x_all = synthetic.make_tokens(tokens, cfg.hidden_size, seed=5)
        per = tokens // world
        x = x_all[rank * per:(rank + 1) * per].contiguous()
        engine = ep.ExpertParallelEngine(NumpyStages(ocfg, ow, rank, world),
                                         capacity_per_rank=capacity)
        out = torch.zeros((per, cfg.hidden_size), dtype=torch.float32)
        engine.step(x, out)
        engine.step(x, out)  # a second step reuses every buffer
        assert capacity > 0 or sum(engine.last_send_splits) == per * cfg.top_k
        np.save(os.path.join(result_dir, f"out{rank}.npy"), out.numpy())
        if rank == 0:
            oracle = entry.load_oracle()
            full = oracle.layer_forward(ocfg, ow, x_all.to(torch.float32).numpy()).out
            np.save(os.path.join(result_dir, "expected.npy"), full)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,tokens,capacity", [(2, 12, 0), (4, 8, 0), (2, 12, 24), (4, 8, 8)])
def test_expert_parallel_protocol_equals_single_process_oracle(tmp_path, world, tokens, capacity):
    """capacity == 0: compact records, split sizes read on the host; capacity > 0: fixed
    segments per destination rank, equal splits, no host round trip."""
    mp.spawn(_worker, args=(world, _free_port(), tokens, str(tmp_path), capacity), nprocs=world,
             join=True)
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    expected = np.load(tmp_path / "expected.npy")
    assert np.array_equal(got, expected)


def test_shard_bindings_splits_experts(package, synthetic):
    ep = importlib.import_module("nemotron_inference_b200.expert_parallel")
    cfg = synthetic.baseline_config(8, experts=32, hidden=64, routed=64, shared=64)
    data = synthetic.make_layer(cfg, seed=1, device="cpu")
    shards = [ep.shard_bindings(data.bindings, r, 4) for r in range(4)]
    assert [s.first_local_expert for s in shards] == [0, 8, 16, 24]
    assert all(len(s.routed_experts) == 8 for s in shards)
    assert shards[2].routed_experts[0] is data.bindings.routed_experts[16]


# --- failure detection on the host side (no GPU involved) -----------------------------

def _faulty_worker(rank, world, port, result_dir, fault):
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=8))
    entry.load_package()
    synthetic = importlib.import_module("nemotron_inference_b200.synthetic")
    ep = importlib.import_module("nemotron_inference_b200.expert_parallel")
    import helpers
    from ep_cpu_stages import NumpyStages
    cfg = synthetic.baseline_config(64, experts=32, hidden=128, routed=64, shared=128, top_k=4)
    data = synthetic.make_layer(cfg, seed=17, device="cpu", norm_weight_uniform=True)
    ocfg, ow = helpers.oracle_config(cfg), helpers.oracle_weights(data)
    x = synthetic.make_tokens(6, cfg.hidden_size, seed=5 + rank)
    stages = NumpyStages(ocfg, ow, rank, world)
    if fault == "wrong_count" and rank == 1:
        honest = stages.dispatch

        def lying_dispatch(x, capacity=0):
            records, counts = honest(x, capacity)
            counts[0] += 1  # claims one more record for rank 0 than it packed
            return records, counts
        stages.dispatch = lying_dispatch
    engine = ep.ExpertParallelEngine(stages)
    out = torch.zeros((6, cfg.hidden_size), dtype=torch.float32)
    outcome = "no error"
    try:
        if fault == "rank_leaves":
            engine.step(x, out)       # a healthy step first
            if rank == 1:
                os._exit(0)           # leaves between steps, without a word
        engine.step(x, out)
    except ep.ExpertParallelError as error:
        outcome = "ExpertParallelError: " + str(error)
    except Exception as error:  # noqa: BLE001 - a timed-out collective raises a backend error
        outcome = type(error).__name__
    with open(os.path.join(result_dir, f"outcome{rank}.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)  # the group is broken by design: no orderly teardown


def test_a_wrong_count_ends_the_step_with_the_same_error_on_every_rank(tmp_path):
    mp.spawn(_faulty_worker, args=(2, _free_port(), str(tmp_path), "wrong_count"), nprocs=2,
             join=True)
    outcomes = [(tmp_path / f"outcome{r}.txt").read_text() for r in range(2)]
    assert outcomes[1].startswith("ExpertParallelError") and "inconsistent" in outcomes[1]
    assert outcomes[0].startswith("ExpertParallelError") and "another rank" in outcomes[0]


@pytest.mark.timeout(60)
def test_a_rank_that_leaves_between_steps_turns_into_an_error_not_a_hang(tmp_path):
    import time
    start = time.time()
    mp.spawn(_faulty_worker, args=(2, _free_port(), str(tmp_path), "rank_leaves"), nprocs=2,
             join=True)
    assert time.time() - start < 45
    outcome = (tmp_path / "outcome0.txt").read_text()
    assert outcome != "no error", outcome  # the survivor's next collective raised
