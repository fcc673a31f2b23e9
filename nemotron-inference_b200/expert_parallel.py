"""Expert-parallel MoE layer: one process per GPU, experts sharded by rank, token
dispatch and return as all-to-all over NCCL.

The reference is single-GPU; this module's contract is "the expert-parallel layer returns
what the single-device layer returns".  Rank r owns experts [r*E/W, (r+1)*E/W) and its own
slice of the tokens; router and shared-expert weights are replicated.

One step (see nmoe_ep_* in include/nmoe.h for the device stages):

    dispatch   route own tokens, pack one record per (token, slot) pair by destination rank
    exchange   per-rank counts (all-to-all), then the records (all-to-all-v)
    experts    local experts over the received records -> one weighted row per record
    shared     shared expert on the own tokens (side stream, overlaps the exchange)
    return     the rows travel back (all-to-all-v, splits swapped)
    combine    out = x + (sum of the token's returned rows in selection order + shared)

The exchange protocol lives in `ExpertParallelEngine`, which is generic over a `stages`
object, so that the protocol itself is testable on CPU with gloo and a numpy stage
implementation; `DeviceStages` is the CUDA implementation over the C ABI.
"""
from __future__ import annotations

import ctypes
import os
import sys
from typing import List, Optional

import torch
import torch.distributed as dist

from . import (ExpertLayerBindings, ExpertLayerConfig, ExpertLayerSlice, NMOE_OK, NmoeError,
               _check, _dtype_code, _stream, load_library)


class DeviceStages:
    """The four device stages of one rank, over libnmoe_b200.so."""

    def __init__(self, config: ExpertLayerConfig, bindings: ExpertLayerBindings, rank: int,
                 world: int, rows_dtype: torch.dtype = torch.float16):
        # config.max_recv_pairs bounds what this rank accepts per step in either layout
        experts_per_rank = config.n_routed_experts // world
        assert len(bindings.routed_experts) == experts_per_rank
        bindings.first_local_expert = rank * experts_per_rank
        self.layer = ExpertLayerSlice.create(config, bindings)
        if self.layer is None:
            raise RuntimeError("expert-parallel layer creation failed: " +
                               ExpertLayerSlice.create_error)
        self.layer.keep_trace(False)  # expert-parallel stages expose no trace
        # the collectives run beside the persistent GEMMs: leave them some SMs
        self.reserved_sms = int(os.environ.get("NMOE_EP_RESERVED_SMS", "16")) if world > 1 else 0
        self.layer.reserve_sms(self.reserved_sms)
        self.config = config
        self.world = world
        self.rows_dtype = rows_dtype
        self.device = torch.device("cuda", torch.cuda.current_device())
        lib = load_library()
        self.record_bytes = int(lib.nmoe_ep_record_bytes(self.layer._handle))
        self.capacity = config.max_recv_pairs or 2 * config.max_tokens * config.top_k
        pairs = config.max_tokens * config.top_k
        H = config.hidden_size
        # exchange buffers are owned here; the library owns only the send records
        self.recv_records = torch.empty((self.capacity, self.record_bytes), dtype=torch.uint8,
                                        device=self.device)
        self.rows_out = torch.empty((self.capacity, H), dtype=rows_dtype, device=self.device)
        self.rows_back = torch.empty((max(pairs, self.capacity), H), dtype=rows_dtype,
                                     device=self.device)
        self.send_slots = 2 * pairs + 64 * 16  # what the library reserves for send records
        self.side_stream = torch.cuda.Stream()
        self._send_view = None

    def dispatch(self, x: torch.Tensor, capacity: int = 0):
        """capacity == 0: compact records (one per pair); capacity > 0: world * capacity
        record slots, destination rank r owning slots [r*capacity, (r+1)*capacity)."""
        lib = load_library()
        records, counts = ctypes.c_void_p(), ctypes.c_void_p()
        _check(lib.nmoe_ep_dispatch(self.layer._handle, _stream(), x.data_ptr(), _dtype_code(x),
                                    x.shape[0], capacity, ctypes.byref(records),
                                    ctypes.byref(counts)),
               "nmoe_ep_dispatch", self.layer._last_error())
        pairs = capacity * self.world if capacity > 0 else x.shape[0] * self.config.top_k
        send_records = _as_tensor(records.value, (pairs, self.record_bytes), torch.uint8,
                                  self.device)
        send_counts = _as_tensor(counts.value, (self.world,), torch.int32, self.device)
        return send_records, send_counts

    def experts(self, recv_records: torch.Tensor, count: int, row_offset: int = 0,
                valid_counts: Optional[torch.Tensor] = None, capacity: int = 0) -> torch.Tensor:
        """Local experts over `count` record slots; row i of the result belongs to slot i.
        With fixed-capacity segments, valid_counts[j] (device int32) says how many of the
        `capacity` slots of segment j hold a record."""
        out = self.rows_out[row_offset:row_offset + count]
        if count > 0:
            _check(load_library().nmoe_ep_experts(
                self.layer._handle, _stream(), recv_records.data_ptr(), count,
                valid_counts.data_ptr() if valid_counts is not None else None, capacity,
                out.data_ptr(), _dtype_code(self.rows_out)),
                "nmoe_ep_experts", self.layer._last_error())
        return out

    def shared(self) -> None:
        """Shared expert over the tokens of the last dispatch, on the compute stream: it keeps
        the GPU busy while the host waits for the split sizes and the records travel."""
        _check(load_library().nmoe_ep_shared(self.layer._handle, _stream()),
               "nmoe_ep_shared", self.layer._last_error())

    def combine(self, x: torch.Tensor, rows_back: torch.Tensor, out: torch.Tensor) -> None:
        _check(load_library().nmoe_ep_combine(self.layer._handle, _stream(), x.data_ptr(),
                                              _dtype_code(x), rows_back.data_ptr(),
                                              _dtype_code(rows_back), out.data_ptr(),
                                              _dtype_code(out)), "nmoe_ep_combine")

    # -- peer windows: the exchanges done by the stages' own kernels over NVLink
    def attach_windows(self, capacity: int, group=None) -> bool:
        """Creates this rank's window, exchanges the handles and maps the peers' windows.
        Every rank takes part in every collective of the set-up whether or not its own
        steps succeeded, so the ranks agree on the outcome: True when all of them are
        attached, False (and nothing left attached) otherwise; `attach_error` says why."""
        lib = load_library()
        handle = (ctypes.c_uint8 * 64)()
        self.attach_error = ""
        status = lib.nmoe_ep_window_create(self.layer._handle, capacity,
                                           _dtype_code(self.rows_out), handle)
        if status != NMOE_OK:
            self.attach_error = f"nmoe_ep_window_create: {self.layer._last_error() or status}"
        gathered = [None] * self.world
        dist.all_gather_object(gathered, (status == NMOE_OK, bytes(handle)), group=group)
        everyone = all(ok for ok, _ in gathered)
        if everyone:
            table = (ctypes.c_uint8 * (64 * self.world)).from_buffer_copy(
                b"".join(h for _, h in gathered))
            status = lib.nmoe_ep_window_attach(self.layer._handle, table)
            if status != NMOE_OK:
                self.attach_error = f"nmoe_ep_window_attach: {self.layer._last_error() or status}"
        outcome = [None] * self.world
        dist.all_gather_object(outcome, everyone and status == NMOE_OK, group=group)
        if not all(outcome):
            lib.nmoe_ep_window_detach(self.layer._handle)
            dist.barrier(group=group)
            return False
        self.window_capacity = capacity
        # the shared expert starts inside the dispatch stage, beside the router kernels
        self.fork_shared = os.environ.get("NMOE_EP_FORK_SHARED", "1") == "1" and \
            lib.nmoe_ep_window_fork_shared(self.layer._handle, 1) == NMOE_OK
        self.layer.reserve_sms(0)  # no collective kernels run beside the GEMMs in this mode
        self.reserved_sms = 0
        dist.barrier(group=group)
        return True

    def detach_windows(self, group=None) -> None:
        torch.cuda.synchronize()
        dist.barrier(group=group)
        _check(load_library().nmoe_ep_window_detach(self.layer._handle), "nmoe_ep_window_detach")
        self.window_capacity = 0
        dist.barrier(group=group)

    def window_dispatch(self, x: torch.Tensor) -> None:
        _check(load_library().nmoe_ep_window_dispatch(self.layer._handle, _stream(), x.data_ptr(),
                                                      _dtype_code(x), x.shape[0]),
               "nmoe_ep_window_dispatch", self.layer._last_error())

    def window_experts(self, first_rank: int, ranks: int) -> None:
        _check(load_library().nmoe_ep_window_experts(self.layer._handle, _stream(), first_rank,
                                                     ranks),
               "nmoe_ep_window_experts", self.layer._last_error())

    def window_combine(self, x: torch.Tensor, out: torch.Tensor) -> None:
        _check(load_library().nmoe_ep_window_combine(self.layer._handle, _stream(), x.data_ptr(),
                                                     _dtype_code(x), out.data_ptr(),
                                                     _dtype_code(out)),
               "nmoe_ep_window_combine", self.layer._last_error())

    # -- optional phase timing: `profile = True` makes mark() record a CUDA event on the
    #    current stream; phase_times_ms() reports them relative to the first mark
    profile = False

    def mark(self, name: str) -> None:
        if self.profile:
            event = torch.cuda.Event(enable_timing=True)
            event.record()
            self._marks.append((name, event))

    def reset_marks(self) -> None:
        self._marks = []

    def phase_times_ms(self) -> dict:
        torch.cuda.synchronize()
        start = self._marks[0][1]
        return {name: start.elapsed_time(event) for name, event in self._marks}

    # -- stream hooks: collectives are issued from a communication stream so that they
    #    depend only on the kernels that produce their inputs
    def comm_stream(self):
        return torch.cuda.stream(self.side_stream)

    def main_to_comm(self) -> None:
        event = torch.cuda.Event()
        event.record()
        self.side_stream.wait_event(event)

    def comm_to_main(self) -> None:
        event = torch.cuda.Event()
        event.record(self.side_stream)
        torch.cuda.current_stream().wait_event(event)

    def count_buffer(self) -> torch.Tensor:
        if not hasattr(self, "_recv_counts"):
            self._recv_counts = torch.zeros((self.world,), dtype=torch.int32, device=self.device)
        return self._recv_counts

    def recv_buffer(self, count: int) -> torch.Tensor:
        if count > self.capacity:
            raise NmoeError(6, "expert-parallel receive",
                            f"{count} pairs exceed the capacity of {self.capacity}")
        return self.recv_records[:count]

    def back_buffer(self, count: int) -> torch.Tensor:
        return self.rows_back[:count]

    def sync_status(self) -> int:
        return self.layer.sync_status()

    def launches_per_window_step(self, groups: int) -> int:
        """Kernels one peer-window step launches on this rank: epoch, the routing front end
        (5), dispatch plan, record packing, flag signal, the shared expert's two GEMMs,
        then per source-rank group wait + histogram + plan + permute + two GEMMs + signal,
        and wait + combine."""
        return 1 + 5 + 3 + 2 + 7 * groups + 2


def _as_tensor(address: int, shape, dtype, device) -> torch.Tensor:
    """A torch view of library-owned device memory (no copy, no ownership)."""
    numel = 1
    for s in shape:
        numel *= s
    itemsize = torch.empty((), dtype=dtype).element_size()

    class _Holder:
        pass

    holder = _Holder()
    holder.__cuda_array_interface__ = {
        "shape": (numel * itemsize,), "typestr": "|u1", "data": (address, False), "version": 3}
    flat = torch.as_tensor(holder, device=device)
    return flat.view(dtype).view(shape)


class ExpertParallelError(RuntimeError):
    """A step cannot go on: some rank reported counts that do not add up, or more pairs
    than a receiver can hold.  Raised on EVERY rank of the group in the same step, before
    any record travels, so no rank is left waiting in a collective."""


class ExpertParallelEngine:
    """The exchange protocol of one rank.  `stages` provides dispatch / experts / shared /
    combine plus recv_buffer / back_buffer; tensors may live on any device the process
    group's backend can move (CUDA with NCCL, CPU with gloo)."""

    def __init__(self, stages, group=None, chunks: Optional[int] = None,
                 capacity_per_rank: int = 0):
        """capacity_per_rank > 0 selects fixed-capacity record segments: all exchanges
        have equal, host-known splits, so a step never synchronises with the host."""
        self.capacity = capacity_per_rank
        self._graph = None
        self.stages = stages
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.chunks = max(1, min(chunks if chunks is not None else 2, self.world))
        self.window_groups = int(os.environ.get("NMOE_EP_WINDOW_GROUPS", "1"))
        self.last_send_splits: List[int] = []
        self.last_recv_splits: List[int] = []

    def step(self, x: torch.Tensor, out: torch.Tensor) -> None:
        if getattr(self.stages, "window_capacity", 0) > 0:
            self._step_window(x, out)
        elif self.capacity > 0:
            self._step_fixed(x, out)
        else:
            self._step_compact(x, out)

    def _step_window(self, x: torch.Tensor, out: torch.Tensor) -> None:
        """Peer-window step: one stream, no collective and no host synchronisation.  The
        shared expert runs while the peers' records are still arriving."""
        st, W = self.stages, self.world
        mark = getattr(st, "mark", lambda name: None)
        mark("start")
        st.window_dispatch(x)
        mark("dispatch_done")
        if not getattr(st, "fork_shared", False):
            st.shared()
        mark("shared_done")
        # the rows travel inside the GEMM's own epilogue, so splitting the source ranks into
        # groups buys no overlap here; one group keeps the launch count and GEMM tails low
        groups = max(1, min(self.window_groups, W))
        bounds = [W * c // groups for c in range(groups + 1)]
        for c in range(groups):
            st.window_experts(bounds[c], bounds[c + 1] - bounds[c])
            mark(f"experts_{c}_done")
        st.window_combine(x, out)
        mark("combine_done")
        cap = st.window_capacity
        self.last_send_splits = self.last_recv_splits = [cap] * W

    def _step_fixed(self, x: torch.Tensor, out: torch.Tensor) -> None:
        st, cap, W = self.stages, self.capacity, self.world
        mark = getattr(st, "mark", lambda name: None)
        mark("start")
        send_records, send_counts = st.dispatch(x, cap)
        mark("dispatch_done")
        st.main_to_comm()
        st.shared()
        mark("shared_done")
        with st.comm_stream():
            recv_counts = st.count_buffer()
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
            recv = st.recv_buffer(W * cap)
            dist.all_to_all_single(recv, send_records, group=self.group)
            mark("records_arrived")
        st.comm_to_main()
        back = st.back_buffer(W * cap)
        bounds = [W * c // self.chunks for c in range(self.chunks + 1)]
        for c in range(self.chunks):
            lo, hi = bounds[c], bounds[c + 1]
            rows = st.experts(recv[lo * cap:hi * cap], (hi - lo) * cap, lo * cap,
                              recv_counts[lo:hi], cap)
            mark(f"experts_{c}_done")
            st.main_to_comm()
            with st.comm_stream():
                in_splits = [cap if lo <= r < hi else 0 for r in range(W)]
                if lo <= self.rank < hi:
                    dist.all_to_all_single(back, rows, [cap] * W, in_splits, group=self.group)
                else:
                    dist.all_to_all_single(back[:0], rows, [0] * W, in_splits, group=self.group)
                mark(f"rows_{c}_returned")
        st.comm_to_main()
        st.combine(x, back, out)
        mark("combine_done")
        self.last_send_splits = self.last_recv_splits = [cap] * W

    def capture(self, x: torch.Tensor, out: torch.Tensor) -> bool:
        """Records one fixed-capacity step on (x, out) as a CUDA graph; `replay` then costs
        one launch.  Returns False (and stays eager) if the capture is not possible."""
        if self.capacity <= 0 and getattr(self.stages, "window_capacity", 0) <= 0:
            return False
        try:
            for _ in range(2):
                self.step(x, out)  # warm up: allocations, NCCL channels
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            # other threads (the NCCL watchdog) make CUDA calls of their own during capture
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                self.step(x, out)
            self._graph = graph
            return True
        except Exception as error:  # noqa: BLE001 - any capture failure means "stay eager"
            self.capture_error = str(error)
            self._graph = None
            torch.cuda.synchronize()
            return False

    def replay(self) -> None:
        self._graph.replay()

    def release_graph(self) -> None:
        """Drops the recorded step.  Do this before the process group is destroyed: a live
        graph keeps the communicator's kernels referenced and the teardown waits for it."""
        if self._graph is not None:
            torch.cuda.synchronize()
            self._graph = None
            import gc
            gc.collect()

    def _step_compact(self, x: torch.Tensor, out: torch.Tensor) -> None:
        st = self.stages
        send_records, send_counts = st.dispatch(x)
        st.main_to_comm()
        st.shared()  # overlaps the host's wait for the split sizes and the dispatch exchange
        with st.comm_stream():
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
            # the split sizes of the variable-size exchange must be known on the host
            both = torch.stack([send_counts, recv_counts]).cpu()
            send_splits = [int(v) for v in both[0]]
            recv_splits = [int(v) for v in both[1]]
            # Every rank checks what it sent and what it was told to expect; the ranks then
            # agree (one small all-reduce) before the variable-size exchange, so that a bad
            # count ends the step with the same error everywhere instead of leaving the
            # healthy ranks inside a collective that can never complete.
            problem = ""
            if min(send_splits + recv_splits) < 0 or sum(send_splits) != send_records.shape[0]:
                problem = f"inconsistent dispatch counts {send_splits}"
            elif sum(recv_splits) > getattr(st, "capacity", sum(recv_splits)):
                problem = f"{sum(recv_splits)} pairs exceed the receive capacity"
            verdict = send_counts.new_tensor([0 if problem else 1])
            dist.all_reduce(verdict, op=dist.ReduceOp.MIN, group=self.group)
            if int(verdict.item()) == 0:
                raise ExpertParallelError(
                    f"rank {self.rank}: " + (problem or "another rank reported bad counts"))
            recv = st.recv_buffer(sum(recv_splits))
            dist.all_to_all_single(recv, send_records, recv_splits, send_splits, group=self.group)
        st.comm_to_main()
        back = st.back_buffer(sum(send_splits))
        # Source ranks are served in contiguous groups: while one group's rows travel home,
        # the next group's records are being computed.
        bounds = [self.world * c // self.chunks for c in range(self.chunks + 1)]
        row_offset = 0
        for c in range(self.chunks):
            lo, hi = bounds[c], bounds[c + 1]
            count = sum(recv_splits[lo:hi])
            rows = st.experts(recv[row_offset:row_offset + count], count, row_offset)
            st.main_to_comm()
            with st.comm_stream():
                in_splits = [recv_splits[r] if lo <= r < hi else 0 for r in range(self.world)]
                if lo <= self.rank < hi:
                    dist.all_to_all_single(back, rows, send_splits, in_splits, group=self.group)
                else:
                    dist.all_to_all_single(back[:0], rows, [0] * self.world, in_splits,
                                           group=self.group)
            row_offset += count
        st.comm_to_main()
        st.combine(x, back, out)
        self.last_send_splits, self.last_recv_splits = send_splits, recv_splits


def shard_bindings(bindings: ExpertLayerBindings, rank: int, world: int) -> ExpertLayerBindings:
    """The bindings of rank `rank`: its slice of the routed experts, everything else shared."""
    per_rank = len(bindings.routed_experts) // world
    return ExpertLayerBindings(
        input_norm_weight=bindings.input_norm_weight, gate_weight=bindings.gate_weight,
        gate_score_correction_bias=bindings.gate_score_correction_bias,
        shared_up=bindings.shared_up, shared_down=bindings.shared_down,
        routed_experts=bindings.routed_experts[rank * per_rank:(rank + 1) * per_rank],
        gate_logit_offset=bindings.gate_logit_offset, first_local_expert=rank * per_rank)


def bench_main(args, package, synthetic, peaks, flush_buf, dist_module, bench_module):
    """bench.py's N > 1 arm: T tokens in total, T / N per rank, experts split over the ranks."""
    import numpy as np
    rank, world = dist_module.get_rank(), dist_module.get_world_size()
    tokens_total = args.tokens
    tokens = tokens_total // world
    H = synthetic.HIDDEN
    cfg = synthetic.baseline_config(max_tokens=tokens)
    # fixed record segments, 25 % above the uniform share: equal exchange splits, no host
    # round trip, and the whole step replays as one CUDA graph
    capacity = segment_capacity(tokens, cfg.top_k, world, worst_case=False)
    cfg.max_recv_pairs = capacity * world
    data = synthetic.make_layer(cfg, seed=4000, device="cuda")
    stages = DeviceStages(cfg, shard_bindings(data.bindings, rank, world), rank, world)
    x_all = synthetic.make_tokens(tokens_total, H, seed=4001)
    # One GPU holding all experts, for two purposes.  (1) Every rank runs it on its own
    # token slice after the timed region and compares the expert-parallel result with it.
    # (2) Rank 0 times it before the ranks start to exchange, on the per-GPU token count
    # (what the exchange and the smaller batches cost) and on all T tokens (the N = 1
    # figure of the strong-scaling efficiency).
    single = package.ExpertLayerSlice.create(synthetic.baseline_config(max_tokens=tokens),
                                             data.bindings)
    if single is None:
        raise SystemExit("single-GPU layer creation failed: " +
                         package.ExpertLayerSlice.create_error)
    single_ms = full_ms = None
    if rank == 0:
        xs = x_all[:tokens].cuda()
        outs = torch.empty((tokens, H), dtype=torch.bfloat16, device="cuda")
        single_ms = float(np.mean(bench_module.time_steps(
            lambda: single.run_async(xs, outs), args.steps, args.warmup, flush_buf)))
        del xs, outs
        full = package.ExpertLayerSlice.create(synthetic.baseline_config(max_tokens=tokens_total),
                                               data.bindings)
        if full is not None:
            xf = x_all.cuda()
            outf = torch.empty((tokens_total, H), dtype=torch.bfloat16, device="cuda")
            full_ms = float(np.mean(bench_module.time_steps(
                lambda: full.run_async(xf, outf), args.steps, args.warmup, flush_buf)))
            full.close()
            del xf, outf
    torch.cuda.empty_cache()
    engine = ExpertParallelEngine(stages, capacity_per_rank=capacity)
    # transport: "window" = the stages' own kernels store into the peers' memory (default);
    # "nccl" = host-issued all-to-all collectives between the stages
    transport = os.environ.get("NMOE_EP_TRANSPORT", "window")
    if transport == "window":
        # peer windows need CUDA IPC between the ranks' processes; where a rank cannot map
        # its peers, every rank falls back to the collectives
        if not stages.attach_windows(capacity):
            print(f"rank {rank}: peer windows unavailable ({stages.attach_error}); using NCCL",
                  file=sys.stderr)
            transport = "nccl"
    x_host = x_all[rank * tokens:(rank + 1) * tokens].contiguous().pin_memory()
    x = x_host.cuda()
    out = torch.empty((tokens, H), dtype=torch.bfloat16, device="cuda")
    out_host = torch.empty((tokens, H), dtype=torch.bfloat16).pin_memory()

    def timed(step_fn, steps, warmup):
        for _ in range(warmup):
            step_fn()
        torch.cuda.synchronize()
        dist_module.barrier()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(steps):
            flush_buf.add_(1)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            step_fn()
            end.record()
            end.synchronize()
            total += start.elapsed_time(end)
        torch.cuda.synchronize()
        dist_module.barrier()
        t = torch.tensor([total / steps], device="cuda")
        dist_module.all_reduce(t, op=dist_module.ReduceOp.MAX)
        return float(t.item())

    ClockSampler, FLOP_PER_TOKEN_TENSOR, METRIC = (bench_module.ClockSampler,
                                                   bench_module.FLOP_PER_TOKEN_TENSOR,
                                                   bench_module.METRIC)
    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    graphed = engine.capture(x, out)
    flags = torch.tensor([1 if graphed else 0], device="cuda")
    dist_module.all_reduce(flags, op=dist_module.ReduceOp.MIN)
    graphed = bool(flags.item())  # every rank replays, or none does
    run_step = engine.replay if graphed else (lambda: engine.step(x, out))
    ms = timed(run_step, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    status = stages.sync_status()
    if status != NMOE_OK:
        raise SystemExit(f"rank {rank}: device error {status}")

    # Correctness of what was just timed, outside the timed region: the output of the
    # last timed step against the single-GPU layer on the same tokens, on every rank; on
    # rank 0 the single-GPU layer against the CPU oracle on the first 256 of them.
    parity = ep_parity_check(package, single, data, x, out, rank, dist_module)
    single.close()
    del data
    torch.cuda.empty_cache()

    def e2e_step():
        x.copy_(x_host, non_blocking=True)
        run_step()
        out_host.copy_(out, non_blocking=True)

    serial_ms = timed(e2e_step, args.steps, args.warmup)
    # pipelined: the recorded step works on fixed buffers, so the pipeline's slots are
    # staged through them with device-to-device copies
    from .host_pipeline import HostPipeline

    def staged_step(x_slot, out_slot):
        x.copy_(x_slot, non_blocking=True)
        run_step()
        out_slot.copy_(out, non_blocking=True)

    pipe = HostPipeline(staged_step, tokens, H)
    local_ms = bench_module.time_pipelined(pipe, x_host, out_host, args.steps, args.warmup,
                                           barrier=dist_module.barrier)
    t = torch.tensor([local_ms], device="cuda")
    dist_module.all_reduce(t, op=dist_module.ReduceOp.MAX)
    e2e_ms = float(t.item())
    stages.profile = True
    phases = {}
    for i in range(4):
        stages.reset_marks()
        flush_buf.add_(1)
        engine.step(x, out)
        if i >= 1:
            for name, ms_at in stages.phase_times_ms().items():
                phases[name] = phases.get(name, 0.0) + ms_at / 3
    stages.profile = False
    engine.release_graph()
    nccl_arm = None
    if transport == "window":
        stages.detach_windows()
        # the configuration as the benchmark definition words it: dispatch and return as
        # NCCL all-to-all, same stages, same fixed segments (eager: collectives between them)
        try:
            stages.layer.reserve_sms(int(os.environ.get("NMOE_EP_RESERVED_SMS", "16")))
            nccl_ms = timed(lambda: engine.step(x, out), max(3, args.steps // 2), 3)
            nccl_arm = {"ms_per_step": nccl_ms, "tokens_per_s": tokens_total / (nccl_ms * 1e-3),
                        "how": "same stages with host-issued NCCL all-to-all of the fixed "
                               "segments between them, eager launches, 16 SMs kept free for "
                               "NCCL's kernels"}
            if stages.sync_status() != NMOE_OK:
                nccl_arm["device_error"] = True
        except Exception as error:  # noqa: BLE001 - an extra key must not lose the line
            nccl_arm = {"unavailable": str(error)[:200]}
    stack_report = None
    if not args.no_side:
        try:
            stack_report = stack_workload(args, package, synthetic, flush_buf, dist_module)
        except Exception as error:  # noqa: BLE001 - a side workload must not lose the line
            stack_report = {"workload": "configs[4]", "unavailable": str(error)[:300]}
    sent = capacity * (world - 1)
    if transport == "window":
        exchange = {
            "dispatch": f"NVFP4 records, {stages.record_bytes} B per pair, stored by the packing "
                        f"kernel straight into the destination GPU's window (fixed segments of "
                        f"{capacity} pairs per (source, destination)); flag words signal arrival",
            "return": "binary16 rows (2 bytes per element, as the bf16 rows of the benchmark "
                      "definition, eight times finer) stored by the down-projection epilogue "
                      "of the grouped GEMM straight into the source GPU's window, tile by tile",
        }
        launches = stages.launches_per_window_step(engine.window_groups)
    else:
        exchange = {
            "dispatch": f"NVFP4 records, {stages.record_bytes} B per pair, fixed segments of "
                        f"{capacity} pairs per (source, destination), NCCL all-to-all",
            "return": "binary16 rows, same segments, NCCL all-to-all in two source-rank groups",
        }
        launches = 13 + 6 * engine.chunks
    value = tokens_total / (ms * 1e-3)
    return {
        "metric": METRIC, "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"configs[3]: T={tokens_total} tokens, uniform routing, hidden 2688, "
                               f"128 experts x 1856 top-6 ({128 // world} per GPU), shared 3712 "
                               "replicated, bf16 in/out",
                   "global_tokens": tokens_total, "parallelism": f"ep{world}",
                   "transport": transport, **exchange,
                   "step_launch": "one CUDA graph replay" if graphed else "eager",
                   "gemm_sms": f"{stages.reserved_sms} SMs kept free of GEMM CTAs for the "
                               "collectives' kernels",
                   "l2": "256 MB buffer written between timed steps; working set > L2"},
        "layer_tflops": tokens_total * FLOP_PER_TOKEN_TENSOR / (ms * 1e-3) / 1e12,
        "e2e": {"value": tokens_total / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": x_host.numel() * 2 * world,
                "d2h_bytes_per_step": out_host.numel() * 2 * world,
                "how": "HostPipeline on every rank: pinned host batches, uploads and downloads "
                       "of neighbouring steps overlap the compute",
                "one_batch_at_a_time_ms_per_step": serial_ms},
        "gpu_launches": launches * args.steps * world,
        "clocks": clocks,
        "ep_parity": parity,
        "per_gpu_tokens": tokens,
        "single_gpu_all_tokens": None if full_ms is None else {
            "what": f"one GPU, all 128 experts, all T={tokens_total} tokens, measured on rank 0 "
                    "in this run",
            "ms_per_step": full_ms, "tokens_per_s": tokens_total / (full_ms * 1e-3)},
        "strong_scaling_efficiency": None if full_ms is None else
        value / (world * tokens_total / (full_ms * 1e-3)),
        "single_gpu_same_tokens": None if single_ms is None else {
            "what": f"one GPU, all 128 experts, T={tokens} (the per-GPU token count of this run)",
            "ms_per_step": single_ms, "tokens_per_s": tokens / (single_ms * 1e-3)},
        "ep_overhead_efficiency_same_per_gpu_tokens": None if single_ms is None else
        value / (world * tokens / (single_ms * 1e-3)),
        "nccl_transport": nccl_arm,
        "also": [stack_report] if stack_report is not None else [],
        "exchange_bytes_rank0": {"dispatch": sent * stages.record_bytes, "return": sent * H * 2},
        "ep_phase_end_ms_rank0_eager": {k: round(v, 4) for k, v in phases.items()},
        "roofline": None,
    }


def segment_capacity(tokens_per_rank: int, top_k: int, world: int, worst_case: bool = True) -> int:
    """Record slots per (source, destination) pair.  worst_case: every pair of a rank may go
    to one destination (tokens_per_rank * top_k slots): no routing can overflow it, which is
    what a stack of real layers needs -- a few layers deep the hidden state routes far from
    uniformly (measured on the synthetic 23-layer stack: one rank's share 39 % above the
    other's, the hottest expert at six times the mean).  Otherwise the uniform share plus a
    quarter, for workloads that route uniformly by construction; a step that needs more
    reports NMOE_ERR_CAPACITY."""
    if worst_case:
        return (tokens_per_rank * top_k + 15) // 16 * 16
    return (int(1.25 * tokens_per_rank * top_k / world) + 15) // 16 * 16


def stack_workload(args, package, synthetic, flush_buf, dist_module, layers: int = 23,
                   parity_layers: int = 2) -> dict:
    """The 23-layer MoE stack of the benchmark definition on all ranks: independently seeded
    layers of the baseline shape (RMSNorm weight ~U(0.9, 1.1)), residual inside every layer,
    FP32 hidden state handed from layer to layer as the reference's caller loop does
    (runtime/src/api/single_token_forward_model.cpp:588-656); a decode batch of 256 tokens
    and one prefill chunk of 4096 tokens, split evenly over the ranks.  The first
    `parity_layers` layers are also checked: expert-parallel result against the single-GPU
    layer on the same input, and that against the CPU oracle, layer by layer with the
    device's output of one layer as the next one's input."""
    import numpy as np
    from .stack import MoeLayerStack
    rank, world = dist_module.get_rank(), dist_module.get_world_size()
    H = synthetic.HIDDEN
    decode_total, prefill_total = 256, 4096
    max_tokens = prefill_total // world
    cfg = synthetic.baseline_config(max_tokens=max_tokens)
    capacity = segment_capacity(max_tokens, cfg.top_k, world)
    cfg.max_recv_pairs = capacity * world
    engines, keep = [], []
    for index in range(layers):
        data = synthetic.make_layer(cfg, seed=6000 + index, device="cuda",
                                    norm_weight_uniform=True)
        stages = DeviceStages(cfg, shard_bindings(data.bindings, rank, world), rank, world)
        if not stages.attach_windows(capacity):
            raise RuntimeError(f"layer {index}: peer windows unavailable: {stages.attach_error}")
        engines.append(ExpertParallelEngine(stages, capacity_per_rank=capacity))
        if index < parity_layers:
            keep.append(data)
        del data
    torch.cuda.empty_cache()
    stack = MoeLayerStack(engines, H, max_tokens)

    def timed(total_tokens):
        tokens = total_tokens // world
        x_all = synthetic.make_tokens(total_tokens, H, seed=6100 + total_tokens)
        x = x_all[rank * tokens:(rank + 1) * tokens].cuda()
        out = torch.empty((tokens, H), dtype=torch.bfloat16, device="cuda")
        graphed = stack.capture(x, out)
        flag = torch.tensor([1 if graphed else 0], device="cuda")
        dist_module.all_reduce(flag, op=dist_module.ReduceOp.MIN)
        graphed = bool(flag.item())
        step = stack.replay if graphed else (lambda: stack.run(x, out))
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        dist_module.barrier()
        total = 0.0
        steps = max(3, args.steps // 2)
        for _ in range(steps):
            flush_buf.add_(1)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            step()
            end.record()
            end.synchronize()
            total += start.elapsed_time(end)
        torch.cuda.synchronize()
        dist_module.barrier()
        t = torch.tensor([total / steps], device="cuda")
        dist_module.all_reduce(t, op=dist_module.ReduceOp.MAX)
        status = torch.tensor([float(stack.sync_status())], device="cuda")
        dist_module.all_reduce(status, op=dist_module.ReduceOp.MAX)
        stack.release_graph()
        ms = float(t.item())
        return {"tokens": total_tokens, "ms_per_stack_pass": ms,
                "tokens_per_s": total_tokens / (ms * 1e-3),
                "launch": "one CUDA graph of all layers" if graphed else "eager",
                "device_status": int(status.item())}

    decode = timed(decode_total)
    prefill = timed(prefill_total)

    # parity, layer by layer, on the decode batch
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(
        os.path.abspath(__file__))), "tests"))
    tokens = decode_total // world
    x_all = synthetic.make_tokens(decode_total, H, seed=6100 + decode_total)
    current = x_all[rank * tokens:(rank + 1) * tokens].cuda()
    worst_vs_single, oracle_ok, summaries, per_layer, statuses = 0.0, True, [], [], []
    for index in range(parity_layers):
        ep_out = torch.empty((tokens, H), dtype=torch.float32, device="cuda")
        # rank 0 spends seconds in the CPU oracle below; the others must not start the next
        # layer's step meanwhile, or their bounded device waits run out before rank 0's
        # records arrive
        torch.cuda.synchronize()
        dist_module.barrier()
        engines[index].step(current, ep_out)
        single = package.ExpertLayerSlice.create(
            synthetic.baseline_config(max_tokens=max(tokens, 64)), keep[index].bindings)
        ref = torch.empty((tokens, H), dtype=torch.float32, device="cuda")
        single.run_async(current, ref)
        torch.cuda.synchronize()
        layer_diff = float((ep_out - ref).abs().max().item())
        per_layer.append(round(layer_diff, 6))
        statuses.append(int(engines[index].stages.sync_status()))
        worst_vs_single = max(worst_vs_single, layer_diff)
        if rank == 0:
            try:
                import helpers  # the test suite's parity report (CPU oracle): checker only
                report = helpers.compare_layer_with_oracle(single, keep[index], current, ref)
                oracle_ok = oracle_ok and report.ok()
                summaries.append(report.summary())
            except Exception as error:  # noqa: BLE001
                oracle_ok = False
                summaries.append(str(error)[:200])
        single.close()
        current = ep_out  # the device's own output feeds the next layer
    worst = torch.tensor([worst_vs_single], device="cuda")
    dist_module.all_reduce(worst, op=dist_module.ReduceOp.MAX)
    okay = torch.tensor([1.0 if oracle_ok else 0.0], device="cuda")
    dist_module.all_reduce(okay, op=dist_module.ReduceOp.MIN)
    worst_status = torch.tensor([float(max(statuses) if statuses else 0)], device="cuda")
    dist_module.all_reduce(worst_status, op=dist_module.ReduceOp.MAX)
    for engine in engines:
        engine.stages.detach_windows()
        engine.stages.layer.close()
    torch.cuda.empty_cache()
    return {"workload": f"configs[4]: {layers} MoE layers, residual + RMSNorm per layer, "
                        f"expert-parallel over {world} GPUs",
            "decode_batch": decode, "prefill_chunk": prefill,
            "segment_capacity": capacity,
            "parity": {"layers_checked": parity_layers, "tokens_per_rank": tokens,
                       "max_abs_vs_single_gpu_all_ranks": float(worst.item()),
                       "max_abs_vs_single_gpu_rank0_by_layer": per_layer,
                       "device_status_max_over_ranks": int(worst_status.item()),
                       "within_2e-2_of_single_gpu": bool(worst.item() <= 2e-2),
                       "single_gpu_vs_oracle_ok": bool(okay.item() == 1.0),
                       "oracle_reports_rank0": summaries}}


def ep_parity_check(package, single, data, x, out, rank, dist_module) -> dict:
    """Compares `out`, the expert-parallel result for this rank's tokens `x`, with the
    single-GPU layer `single` (all experts, same weights) on the same tokens, and on rank 0
    the single-GPU layer with the CPU oracle on the first 256 tokens.  Returns the record
    rank 0 prints; every rank takes part in the reductions."""
    import numpy as np
    tokens, H = x.shape
    ref = torch.empty((tokens, H), dtype=out.dtype, device=x.device)
    single.run_async(x, ref)
    torch.cuda.synchronize()
    status = single.sync_status()
    diff = (out.to(torch.float32) - ref.to(torch.float32)).abs()
    # bf16 rows: both sides round the same FP32 values, so equality is expected; the gate
    # is the layer tolerance plus half a bf16 ulp at the reference value
    mag = ref.to(torch.float32).abs().clamp_min(2.0 ** -126)
    half_ulp = torch.exp2(torch.floor(torch.log2(mag)) - 8)
    excess = float((diff - half_ulp).max().item())
    stats = torch.tensor([float(torch.equal(out, ref)), -float(diff.max().item()), -excess,
                          float(status == NMOE_OK)], device=x.device, dtype=torch.float64)
    dist_module.all_reduce(stats, op=dist_module.ReduceOp.MIN)
    record = {"tokens_checked_per_rank": tokens,
              "bit_equal_to_single_gpu_on_every_rank": bool(stats[0].item() == 1.0),
              "max_abs_vs_single_gpu": -float(stats[1].item()),
              "within_2e-2_of_single_gpu": bool(-float(stats[2].item()) <= 2e-2),
              "single_gpu_status_ok": bool(stats[3].item() == 1.0)}
    if rank == 0:
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(
            os.path.abspath(__file__))), "tests"))
        try:
            import helpers  # the test suite's parity report (CPU oracle): checker only
            sample = min(256, tokens)
            xs = x[:sample].contiguous()
            outs = torch.empty((sample, H), dtype=torch.float32, device=x.device)
            single.run_async(xs, outs)
            torch.cuda.synchronize()
            report = helpers.compare_layer_with_oracle(single, data, xs, outs)
            record["single_gpu_vs_oracle"] = {"tokens": sample, "ok": bool(report.ok()),
                                              "summary": report.summary()}
        except Exception as error:  # noqa: BLE001
            record["single_gpu_vs_oracle"] = {"ok": False, "error": str(error)[:300]}
    oracle_ok = torch.tensor([1.0 if rank != 0 or record["single_gpu_vs_oracle"]["ok"] else 0.0],
                             device=x.device)
    dist_module.all_reduce(oracle_ok, op=dist_module.ReduceOp.MIN)
    record["ok"] = bool(record["within_2e-2_of_single_gpu"] and record["single_gpu_status_ok"]
                        and oracle_ok.item() == 1.0)
    return record
