"""GPU test of nmoe_route_tokens_noalloc, the routing entry point for callers that must
not allocate device memory when they route (memory handed out once from an arena, a
serving loop that cannot afford an allocation to stall or fail).  Its intermediates live
in a fixed array inside the library, shared by all calls and never cleared, so the test
makes two calls in a row with different shapes and checks each against the three existing
entry points it replaces (nmoe_rmsnorm, nmoe_router_logits, nmoe_router_topk), whose
intermediates are ordinary caller-owned tensors.  Collected last on purpose."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(rows, hidden, experts, seed, dtype):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((rows, hidden), generator=g, device="cuda").to(dtype)
    norm = torch.rand((hidden,), generator=g, device="cuda") * 0.2 + 0.9
    gate = (torch.randn((experts, hidden), generator=g, device="cuda") * 0.02).to(
        torch.bfloat16).to(torch.float32)
    bias = torch.rand((experts,), generator=g, device="cuda") * 0.02 - 0.01
    return x, norm, gate, bias


def _existing_path(package, x, norm, gate, bias, top_k, scaling):
    y = package.rmsnorm(x, norm, 1e-5)
    logits = package.router_logits(y, gate)
    return package.router_topk(logits, bias, top_k, 1, 1, True, scaling)


def test_noalloc_routing_matches_existing_entry_points_twice(package, oracle):
    # first call: many rows; second call: fewer rows and another width, so that stale
    # contents of the shared array from the first call lie beside and behind the second's
    for rows, hidden, experts, top_k, dtype, seed in [
            (300, 2688, 128, 6, torch.bfloat16, 1), (17, 1024, 256, 8, torch.float32, 2)]:
        x, norm, gate, bias = _inputs(rows, hidden, experts, seed, dtype)
        idx, wt = package.route_tokens_noalloc(x, norm, 1e-5, gate, bias, top_k,
                                               routed_scaling=2.5)
        ref_idx, ref_wt = _existing_path(package, x, norm, gate, bias, top_k, 2.5)
        torch.cuda.synchronize()
        assert torch.equal(idx, ref_idx)
        assert torch.equal(wt, ref_wt)  # same kernels, same inputs: not merely within 1e-5
        # and against the CPU restatement of the reference's host path itself
        y = oracle.rmsnorm(x.to(torch.float32).cpu().numpy(), norm.cpu().numpy(), 1e-5)
        o_idx, o_wt = oracle.select_top_experts(
            oracle.router_logits(y, gate.cpu().numpy()), bias.cpu().numpy(), top_k,
            routed_scaling=2.5)
        assert (idx.cpu().numpy() == o_idx).all()
        assert abs(wt.cpu().numpy() - o_wt).max() <= 1.2e-7


def test_noalloc_routing_rejects_sizes_beyond_its_fixed_scratch(package):
    x, norm, gate, bias = _inputs(400, 2688, 128, 3, torch.bfloat16)  # 400 * 2688 > 1,048,576
    with pytest.raises(package.NmoeError) as info:
        package.route_tokens_noalloc(x, norm, 1e-5, gate, bias, 6)
    assert info.value.status == 6  # NMOE_ERR_CAPACITY
