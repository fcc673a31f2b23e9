"""GPU parity tests of the memory-bound stages, through the C ABI, against the CPU oracle:
bit-exact packed FP4 bytes, E4M3 block scales, tensor scales, scale re-tiling, RMSNorm and
router top-k index sets."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _np(t):
    return t.detach().cpu().numpy()


@pytest.mark.parametrize("rows,cols,scale,dtype", [
    (64, 2688, 1.0, torch.bfloat16), (5, 1856, 25.0, torch.float32),
    (3, 3712, 3000.0, torch.float32), (1, 16, 1.0, torch.float32), (130, 64, 1e-4, torch.float32)])
def test_quantiser_is_byte_identical_per_row(package, oracle, rows, cols, scale, dtype):
    g = torch.Generator(device="cuda").manual_seed(rows * 7 + cols)
    x = (torch.randn((rows, cols), generator=g, device="cuda") * scale).to(dtype)
    x[0, :16] = 0
    packed, scales, ts, sw = package.quantize_nvfp4(x, per_row=True, swizzled=True)
    torch.cuda.synchronize()
    op, os_, ots = oracle.pack_nvfp4_per_row(_np(x.to(torch.float32)))
    assert np.array_equal(_np(packed), op)
    assert np.array_equal(_np(scales), os_)
    assert np.array_equal(_np(ts), ots)
    assert np.array_equal(_np(sw), oracle.swizzle_scales(os_, cols))


def test_quantiser_whole_matrix_semantics(package, oracle):
    # device_nvfp4_matrix_test.cpp:26-78: ((i % 11) - 5) * 0.25 and 16 x 4096.0
    a = ((torch.arange(32) % 11) - 5).to(torch.float32).reshape(2, 16) * 0.25
    b = torch.cat([torch.full((1, 16), 4096.0), torch.randn(1, 16)])
    for x in (a, b):
        packed, scales, ts = package.quantize_nvfp4(x.cuda(), per_row=False)
        torch.cuda.synchronize()
        op, os_, ots = oracle.pack_nvfp4(x.numpy())
        assert np.array_equal(_np(packed), op) and np.array_equal(_np(scales), os_)
        assert np.float32(_np(ts)[0]) == np.float32(ots)


def test_decode_of_every_code(package, oracle):
    # all 16 E2M1 codes under all 254 finite E4M3 scale codes (positive and negative)
    scale_codes = np.array([c for c in range(256) if (c & 0x7f) != 0x7f], dtype=np.uint8)
    rows = scale_codes.size
    packed = np.tile(np.array([0x10, 0x32, 0x54, 0x76, 0x98, 0xba, 0xdc, 0xfe], np.uint8), (rows, 1))
    scales = scale_codes.reshape(rows, 1)
    ts = np.float32(0.37)
    out = package.dequant_nvfp4(torch.from_numpy(packed).cuda(), torch.from_numpy(scales).cuda(),
                                torch.tensor([ts], device="cuda"), per_row=False)
    torch.cuda.synchronize()
    expect = oracle.dequant_nvfp4(packed, scales, float(ts))
    assert np.array_equal(_np(out).view(np.uint32), expect.view(np.uint32))


def test_swizzle_matches_oracle(package, oracle):
    rng = np.random.default_rng(3)
    for rows, cols in [(16, 64), (130, 112), (1856, 2688)]:
        sc = rng.integers(0, 127, (rows, cols // 16), dtype=np.uint8)
        out = package.swizzle_scales(torch.from_numpy(sc).cuda(), cols)
        torch.cuda.synchronize()
        assert np.array_equal(_np(out), oracle.swizzle_scales(sc, cols))


@pytest.mark.parametrize("rows,hidden,dtype", [(64, 2688, torch.bfloat16), (7, 4096, torch.float32),
                                               (3, 64, torch.float32)])
def test_rmsnorm_is_bit_identical_to_oracle(package, oracle, rows, hidden, dtype):
    g = torch.Generator(device="cuda").manual_seed(hidden)
    x = torch.randn((rows, hidden), generator=g, device="cuda").to(dtype)
    w = torch.rand((hidden,), generator=g, device="cuda") * 0.2 + 0.9
    y = package.rmsnorm(x, w, 1e-5)
    torch.cuda.synchronize()
    expect = oracle.rmsnorm(_np(x.to(torch.float32)), _np(w), 1e-5)
    assert np.array_equal(_np(y).view(np.uint32), expect.view(np.uint32))
    # and within the reference's own tolerance of a plain float64 evaluation
    # (primitive_ops_test.cpp:105 uses 1e-4)
    x64 = _np(x.to(torch.float32)).astype(np.float64)
    ref = x64 / np.sqrt((x64 ** 2).mean(axis=1, keepdims=True) + 1e-5) * _np(w).astype(np.float64)
    assert np.max(np.abs(_np(y) - ref)) < 1e-5


@pytest.mark.parametrize("rows", [1, 8, 64, 300])
def test_router_logits_and_topk_match_oracle(package, oracle, rows):
    g = torch.Generator(device="cuda").manual_seed(rows)
    E, H, k = 128, 2688, 6
    y = torch.randn((rows, H), generator=g, device="cuda")
    gate = (torch.randn((E, H), generator=g, device="cuda") * 0.02).to(torch.bfloat16).to(torch.float32)
    bias = torch.rand((E,), generator=g, device="cuda") * 0.02 - 0.01
    logits = package.router_logits(y, gate)
    idx, wt = package.router_topk(logits, bias, k, 1, 1, True, 2.5)
    torch.cuda.synchronize()
    expect_logits = oracle.router_logits(_np(y), _np(gate))
    assert np.array_equal(_np(logits).view(np.uint32), expect_logits.view(np.uint32))
    eidx, ewt = oracle.select_top_experts(expect_logits, _np(bias), k, 1, 1, True, 2.5)
    assert np.array_equal(np.sort(_np(idx), axis=1), np.sort(eidx, axis=1))
    assert np.array_equal(_np(idx), eidx)
    assert np.max(np.abs(_np(wt) - ewt)) <= 1e-5  # selection-weight tolerance of expert_layer_oracle_test.cpp


def test_router_topk_grouped_and_wide(package, oracle):
    rng = np.random.default_rng(5)
    for (T, E, k, ng, tg, norm) in [(12, 64, 4, 8, 3, True), (9, 512, 22, 1, 1, True),
                                    (5, 32, 32, 4, 4, False), (6, 256, 8, 8, 4, True)]:
        logits = rng.normal(0, 1, (T, E)).astype(np.float32)
        bias = rng.uniform(-0.01, 0.01, E).astype(np.float32)
        idx, wt = package.router_topk(torch.from_numpy(logits).cuda(), torch.from_numpy(bias).cuda(),
                                      k, ng, tg, norm, 5.0)
        torch.cuda.synchronize()
        eidx, ewt = oracle.select_top_experts(logits, bias, k, ng, tg, norm, 5.0)
        assert np.array_equal(_np(idx), eidx)
        assert np.max(np.abs(_np(wt) - ewt)) <= 1e-5


def test_entry_points_reject_bad_arguments(package):
    x = torch.zeros((2, 15), device="cuda")
    with pytest.raises(package.NmoeError):
        package.quantize_nvfp4(x)
    with pytest.raises(package.NmoeError):
        package.router_topk(torch.zeros((1, 48), device="cuda"), torch.zeros(48, device="cuda"), 6)
