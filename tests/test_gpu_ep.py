"""Multi-GPU test of the expert-parallel layer (needs >= 2 GPUs, skipped otherwise): NCCL
ranks as child processes, exchanging through collectives and through peer windows; every rank also runs the single-device layer over all tokens and
checks that its slice of the expert-parallel output is identical (FP32 return rows) or within
the layer tolerance (bf16 return rows)."""
import importlib
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, shape, tokens_per_rank):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    import datetime
    import faulthandler
    import sys
    import traceback
    faulthandler.dump_traceback_later(100, exit=True, file=sys.stderr)  # a hung rank says where
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=90))
    try:
        package = entry.load_package()
        synthetic = importlib.import_module("nemotron_inference_b200.synthetic")
        ep = importlib.import_module("nemotron_inference_b200.expert_parallel")
        experts, hidden, routed, shared = shape
        total = tokens_per_rank * world
        cfg = synthetic.baseline_config(total, experts=experts, hidden=hidden, routed=routed,
                                        shared=shared)
        data = synthetic.make_layer(cfg, seed=31, device="cuda", norm_weight_uniform=True)
        single = package.ExpertLayerSlice.create(cfg, data.bindings)
        x_all = synthetic.make_tokens(total, hidden, seed=9, device="cuda")
        expected = torch.empty((total, hidden), dtype=torch.float32, device="cuda")
        assert single.run(x_all, expected), single.last_error
        expected_bf16 = torch.empty((total, hidden), dtype=torch.bfloat16, device="cuda")
        assert single.run(x_all, expected_bf16), single.last_error
        mine = slice(rank * tokens_per_rank, (rank + 1) * tokens_per_rank)
        x = x_all[mine].contiguous()
        # compact records (host reads the split sizes) and fixed-capacity segments (no host
        # round trip; replayed as a CUDA graph when the capture succeeds)
        # ... and the same fixed segments exchanged through peer windows: the packing kernel
        # and the GEMM epilogue store into the other GPU's memory, no collective runs
        fixed = 2 * tokens_per_rank * cfg.top_k // world
        # binary16 rows with a bf16 result are what the single-device layer keeps for a bf16
        # result too: that combination must agree bit for bit as well
        for rows_dtype, capacity, window, out_dtype in (
                (torch.float32, 0, False, torch.float32), (torch.bfloat16, 0, False, torch.float32),
                (torch.float32, fixed, False, torch.float32),
                (torch.float32, fixed, True, torch.float32),
                (torch.bfloat16, fixed, True, torch.float32),
                (torch.float16, fixed, True, torch.bfloat16)):
            ep_cfg = synthetic.baseline_config(tokens_per_rank, experts=experts, hidden=hidden,
                                               routed=routed, shared=shared)
            ep_cfg.max_recv_pairs = total * cfg.top_k
            stages = ep.DeviceStages(ep_cfg, ep.shard_bindings(data.bindings, rank, world), rank,
                                     world, rows_dtype=rows_dtype)
            engine = ep.ExpertParallelEngine(stages, capacity_per_rank=capacity)
            if window:
                assert stages.attach_windows(capacity), stages.attach_error
            out = torch.empty((tokens_per_rank, hidden), dtype=out_dtype, device="cuda")
            exact = rows_dtype == torch.float32 or out_dtype == torch.bfloat16
            want = (expected_bf16 if out_dtype == torch.bfloat16 else expected)[mine]
            for _ in range(2):
                engine.step(x, out)
            torch.cuda.synchronize()
            if capacity > 0:
                if exact:
                    assert torch.equal(out, want)
                graphed = engine.capture(x, out)
                flag = torch.tensor([1 if graphed else 0], device="cuda")
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                if flag.item():
                    out.zero_()
                    engine.replay()
                    torch.cuda.synchronize()
                elif rank == 0:
                    print("graph capture unavailable:", getattr(engine, "capture_error", ""))
            assert stages.sync_status() == 0
            if exact:
                assert torch.equal(out, want), (out.float() - want.float()).abs().max().item()
            else:
                assert (out - want).abs().max().item() <= 2e-2
            engine.release_graph()
            if window:
                stages.detach_windows()
            stages.layer.close()
        single.close()
    except BaseException:
        # leave at once: tearing the process group down while the peer sits in a
        # collective would block both ranks until the timeout
        traceback.print_exc()
        os._exit(1)
    dist.destroy_process_group()


@pytest.mark.timeout(150)
@pytest.mark.parametrize("tokens_per_rank", [24, 700])
def test_expert_parallel_equals_single_device(tokens_per_rank):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    mp.spawn(_worker, args=(world, _free_port(), (32, 512, 256, 512), tokens_per_rank),
             nprocs=world, join=True)


def _timeout_worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    import datetime
    import time
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=60))
    outcome = "unfinished"
    try:
        entry.load_package()
        synthetic = importlib.import_module("nemotron_inference_b200.synthetic")
        ep = importlib.import_module("nemotron_inference_b200.expert_parallel")
        tokens = 24
        cfg = synthetic.baseline_config(tokens, experts=32, hidden=512, routed=256, shared=512)
        cfg.max_recv_pairs = tokens * world * cfg.top_k
        data = synthetic.make_layer(cfg, seed=31, device="cuda")
        stages = ep.DeviceStages(cfg, ep.shard_bindings(data.bindings, rank, world), rank, world)
        capacity = 2 * tokens * cfg.top_k // world
        engine = ep.ExpertParallelEngine(stages, capacity_per_rank=capacity)
        assert stages.attach_windows(capacity), stages.attach_error
        x = synthetic.make_tokens(tokens, cfg.hidden_size, seed=9 + rank, device="cuda")
        out = torch.empty((tokens, cfg.hidden_size), dtype=torch.float32, device="cuda")
        engine.step(x, out)                       # a healthy step
        torch.cuda.synchronize()
        assert stages.sync_status() == 0
        dist.barrier()
        # step 2: rank 1 does not take part (between steps, nothing of its own in flight);
        # rank 0's kernels wait for flags that nobody raises, give up after the limit and
        # leave an error status.  Rank 1 stays alive, with its window mapped, until rank 0
        # is done.
        stages.layer.set_wait_limit_ms(50.0)
        if rank == 0:
            start = time.perf_counter()
            engine.step(x, out)
            status = stages.sync_status()
            elapsed = time.perf_counter() - start
            outcome = f"status={status} elapsed={elapsed:.3f}"
        else:
            outcome = "skipped the step"
        dist.barrier()
        stages.detach_windows()
        stages.layer.close()
    except BaseException as error:  # noqa: BLE001
        outcome = "exception: " + repr(error)
    with open(os.path.join(result_dir, f"outcome{rank}.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)


@pytest.mark.timeout(150)
def test_a_peer_that_skips_a_step_costs_a_timeout_status_not_a_hang(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    mp.spawn(_timeout_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    survivor = (tmp_path / "outcome0.txt").read_text()
    assert survivor.startswith("status=4 "), survivor     # NMOE_ERR_DEVICE_TIMEOUT
    assert float(survivor.split("elapsed=")[1]) < 5.0, survivor
    assert (tmp_path / "outcome1.txt").read_text() == "skipped the step"
