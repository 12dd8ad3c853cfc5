"""Numeric primitives: value codec, Oja tracker, index codecs, rank controllers, metrics, accounting."""

import math

import pytest
import torch

from stacr_b200 import cosine_similarity, quantize_values, relative_mse, saved_surface_predictor, stacr_stored_bytes
from stacr_b200.analysis import gradient_bridge, residual_proxy_gain, surface_ledger
from stacr_b200.compressor import STACRCompressor, STACRConfig, stacr_saved_tensors
from stacr_b200.index_compression import (
    BlockOffsetEncoding, DeltaEncodedIndices, IndexCompressionStats, analyze_delta_compression_potential, compress_activation_to_csr,
    compress_indices, csr_memory_savings, decompress_indices, estimate_index_compression, index_dtype_recommendation,
    should_use_delta_encoding, timed_roundtrip,
)
from stacr_b200.oja import OjaBasis, oja_step, orthonormalize
from stacr_b200.quant import pack_int4, unpack_int4
from stacr_b200.rank_controller import choose_runtime_rank, choose_sensitivity_rank, choose_variance_rank, should_adjust_rank
from stacr_b200.residual import select_topk_residual
from stacr_b200.utils import parse_override


def test_int4_pack_roundtrip_and_layout():
    v = torch.tensor([-8, 7, 3, -1, 5], dtype=torch.int8)
    packed = pack_int4(v)
    assert packed.dtype == torch.uint8 and packed.numel() == 3
    assert int(packed[0]) == ((7 & 0xF) << 4) | (-8 & 0xF)
    assert torch.equal(unpack_int4(packed, 5), v)


@pytest.mark.parametrize("bits", [0, 4, 8])
def test_quantize_values_error_bound_and_scale_dtype(bits):
    torch.manual_seed(0)
    v = torch.randn(1001).half()
    q = quantize_values(v, bits)
    assert q.scale.dtype == torch.float32 and q.scale.ndim == 0 and q.length == 1001
    back = q.dequantize(torch.float32)
    if bits == 0:
        assert torch.equal(back, v.float())
    else:
        assert (back - v.float()).abs().max() <= q.scale / 2 + 1e-6
    zero = quantize_values(torch.zeros(4), bits or 8)
    assert torch.equal(zero.dequantize(torch.float32), torch.zeros(4))
    with pytest.raises(ValueError):
        quantize_values(v, 3)


def test_oja_tracks_a_planted_subspace():
    torch.manual_seed(1)
    n, r = 48, 3
    u = orthonormalize(torch.randn(n, r))
    basis = OjaBasis(n, r)
    assert not basis.initialized
    for _ in range(150):
        x = torch.randn(64, r) @ u.t() * 3 + 0.05 * torch.randn(64, n)
        basis.update(x, lr=0.05)
    q = basis.basis
    torch.testing.assert_close(q.t() @ q, torch.eye(r), atol=1e-5, rtol=0)
    assert (u.t() @ q).norm() ** 2 / r > 0.98
    first = basis.shared()
    basis.update(torch.randn(8, n))
    assert basis.shared() is not first  # rebind, never mutate
    stepped = oja_step(q, torch.randn(16, n), 0.01)
    torch.testing.assert_close(stepped.t() @ stepped, torch.eye(r), atol=1e-5, rtol=0)


@pytest.mark.parametrize("mode", ["none", "csr", "delta"])
@pytest.mark.parametrize("preserve", [True, False])
def test_index_codecs_roundtrip(mode, preserve):
    torch.manual_seed(2)
    rows, n = 64, 300
    idx = torch.randperm(rows * n)[:500].to(torch.int32)
    packed = compress_indices(idx, rows, n, mode, preserve_order=preserve)
    back = decompress_indices(packed)
    if preserve or mode == "none":
        assert torch.equal(back, idx)
    else:
        assert torch.equal(back.sort().values, idx.sort().values)
    if mode == "csr":
        assert packed.col_indices.dtype == torch.int16 and packed.row_ptrs.numel() == rows + 1
    empty = compress_indices(idx[:0], rows, n, mode)
    assert decompress_indices(empty).numel() == 0
    est = estimate_index_compression(rows, n, 500, mode, preserve_order=preserve)
    assert est["compressed_bytes"] > 0 and est["mode"] == mode


@pytest.mark.parametrize("mode", ["csr", "delta"])
def test_indices_beyond_int32_roundtrip(mode):
    idx = torch.tensor([2**31 + 15, 2**32 - 1, 2**31 + 2], dtype=torch.int64)
    assert torch.equal(decompress_indices(compress_indices(idx, 4, 2**30, mode)), idx)


def test_index_helpers():
    s = csr_memory_savings(100, 100, 50)
    assert s["dense_bytes"] == 40000 and s["csr_bytes"] == 101 * 4 + 50 * 8
    a = torch.tensor([[0.0, 2.0, 0.0], [1.0, 0.0, -3.0]])
    assert torch.equal(compress_activation_to_csr(a, 0.5).to_dense(), a)
    sorted_idx = torch.arange(0, 4000, 4)
    info = analyze_delta_compression_potential(sorted_idx)
    assert info["avg_delta"] == 4 and info["delta_histogram"]["< 128 (1 byte)"] == 999
    assert should_use_delta_encoding(sorted_idx)
    enc = DeltaEncodedIndices(torch.tensor([9, 3, 70000, 12]))
    assert torch.equal(enc.decode(), torch.tensor([3, 9, 12, 70000], dtype=torch.int32))
    t = torch.zeros(8, 16)
    t[1, 3], t[5, 9] = 2.0, -1.0
    blk = BlockOffsetEncoding(t, 16)
    assert torch.equal(blk.to_dense(), t) and blk.compression_ratio() > 1
    stats = IndexCompressionStats()
    timed_roundtrip(sorted_idx.int(), 1, 4000, "delta", stats)
    assert stats.report()["num_operations"] == 1
    assert index_dtype_recommendation(100) == torch.int8 and index_dtype_recommendation(10**6) == torch.int32
    assert index_dtype_recommendation(100, "speed") == torch.int32


def test_rank_controllers():
    assert should_adjust_rank(5, -1, 100) and not should_adjust_rank(50, 0, 100) and should_adjust_rank(100, 0, 100)
    d = choose_variance_rank([9.0, 0.5, 0.3, 0.2], 4, 1, 8, 4, 0.9)
    assert d.active_rank == 1 and d.reason_code == "variance_shrink" and d.changed
    assert choose_variance_rank(None, 4, 1, 8, 4, 0.9).reason_code == "variance_cold_start"
    assert choose_variance_rank([0.0, 0.0], 4, 2, 8, 4, 0.9).active_rank == 2
    with pytest.raises(ValueError):
        choose_variance_rank([float("nan")], 4, 1, 8, 4, 0.9)
    assert choose_sensitivity_rank(0.2, 8, 4, 32, 32, 0.03, 0.1, 0.125).active_rank == 9
    assert choose_sensitivity_rank(0.01, 8, 4, 32, 32, 0.03, 0.1, 0.125).active_rank == 7
    assert choose_sensitivity_rank(0.05, 8, 4, 32, 32, 0.03, 0.1, 0.125).reason_code == "sensitivity_keep_band"
    assert choose_runtime_rank("fixed", 40, 4, 32, 64, {}).active_rank == 32
    assert choose_runtime_rank("sensitivity", 8, 4, 32, 32, {"last_residual_energy": 0.5}).active_rank == 9
    with pytest.raises(ValueError):
        choose_runtime_rank("other", 8, 4, 32, 32, {})


def test_metrics_edge_cases():
    z = torch.zeros(4)
    assert float(cosine_similarity(z, z)) == 1.0
    assert float(cosine_similarity(z, torch.ones(4))) == 0.0
    tiny = torch.tensor([1e-30, 2e-30])
    assert float(cosine_similarity(tiny, tiny * 3)) == pytest.approx(1.0)
    with pytest.raises(ValueError):
        cosine_similarity(torch.ones(3), torch.ones(4))
    with pytest.raises(ValueError):
        cosine_similarity(torch.tensor([float("inf")]), torch.ones(1))
    assert float(relative_mse(torch.ones(4), torch.ones(4) * 1.1)) == pytest.approx(0.01, rel=1e-4)


def test_byte_accounting():
    assert stacr_stored_bytes((128, 64), 8, torch.float16, 0.01) == 128 * 8 * 2 + 82 * 4 + 82 * 2
    assert stacr_stored_bytes((128, 64), 8, torch.float16, 0.01, residual_bits=8, coeff_bits=8) == 128 * 8 + 4 + 82 * 4 + 82 + 4
    assert stacr_stored_bytes((128, 64), 8, torch.float16, 0.0, include_basis=True, basis_dtype=torch.float32) == 128 * 8 * 2 + 64 * 8 * 4
    assert saved_surface_predictor(50.0, 200.0) == 0.25 and saved_surface_predictor(-5, 10) == 0.0
    with pytest.raises(ValueError):
        saved_surface_predictor(1, 0)
    from stacr_b200.memory import payload_ledger

    items = payload_ledger((128, 64), 8, torch.float16, 0.01, include_basis=True, coeff_bits=8, residual_bits=4)
    assert items == (128 * 8, 82 * 4, 41, 8, 64 * 8 * 2) and items.total == stacr_stored_bytes((128, 64), 8, torch.float16, 0.01, include_basis=True, coeff_bits=8, residual_bits=4)
    assert payload_ledger((), 8).total == 2 and payload_ledger((5, 0), 8).total == 0
    ledger = surface_ledger(1000, 100, 10000, basis_bytes=50, workspace_bytes=20)
    assert ledger["ssp"] == 0.09 and ledger["net_after_workspace_bytes"] == 830


def test_gradient_bridge_inequality_and_gain():
    torch.manual_seed(3)
    a = torch.randn(32, 16)
    rec = a + 0.05 * torch.randn_like(a)
    g = torch.randn(32, 8)
    out = gradient_bridge(a, rec, g)
    assert out["bridge_holds"] and out["cosine_bound_holds"] and out["cosine"] > 0.99
    assert gradient_bridge(a, rec, g, spectral=False)["upstream_norm"] == "frobenius"
    assert residual_proxy_gain(0.99, 0.98) == pytest.approx(1 - ((0.01 / 1.99) / (0.02 / 1.98)) ** 2)
    with pytest.raises(ValueError):
        residual_proxy_gain(1.5, 0.5)


def test_hook_path_compresses_activations_not_parameters():
    torch.manual_seed(4)
    w = torch.nn.Parameter(torch.randn(7, 64))
    comp = STACRCompressor(STACRConfig(min_features=1, min_numel=1, rank=4, residual_budget=0.05))
    assert not comp.should_compress(w.t())
    x = torch.randn(32, 64, requires_grad=True)
    with stacr_saved_tensors(comp):
        y = (x * 2.0).tanh() @ w.t()
    y.sum().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()
    r = select_topk_residual(torch.tensor([[0.1, -5.0], [2.0, 0.0]]), 0.5)
    assert sorted(r.indices.tolist()) == [1, 2] and r.dense(device="cpu", dtype=torch.float32)[0, 1] == -5.0


def test_override_parsing_keeps_on_off_as_strings():
    assert parse_override("true") is True and parse_override("False") is False
    assert parse_override("on") == "on" and parse_override("yes") == "yes" and parse_override("off") == "off"
    assert parse_override("3") == 3 and parse_override("1e-3") == pytest.approx(1e-3) or isinstance(parse_override("1e-3"), (float, str))
    assert parse_override("null") is None and parse_override("[a, on]") == ["a", "on"]
    assert math.isclose(parse_override("0.5"), 0.5)


def test_attention_helpers_on_cpu():
    """Layout helpers and the fp32 formula used as the oracle of the attention kernels (the kernels themselves need a B200)."""
    import torch

    from stacr_b200.ops import attention, nn_ops

    b, s, h, d = 2, 6, 3, 8
    torch.manual_seed(0)
    qkv = torch.randn(b * s, 3 * h * d)
    qi, ki, vi = attention.qkv_views(qkv, b, s, h, d, "interleaved")
    qb, kb, vb = attention.qkv_views(qkv, b, s, h, d, "blocked")
    assert qi.shape == qb.shape == (b, h, s, d)
    # both are views into the same storage, at the columns their layout names
    assert qi.data_ptr() == qkv.data_ptr() and ki.data_ptr() == qkv.data_ptr() + d * 4 and vb.data_ptr() == qkv.data_ptr() + 2 * h * d * 4
    assert torch.equal(qi[1, 2, 3], qkv[1 * s + 3, 2 * 3 * d: 2 * 3 * d + d]) and torch.equal(kb[1, 2, 3], qkv[1 * s + 3, h * d + 2 * d: h * d + 3 * d])
    ref = attention.reference(qi, ki, vi, causal=True)
    want = torch.nn.functional.scaled_dot_product_attention(qi, ki, vi, is_causal=True).transpose(1, 2).reshape(b, s, h * d)
    torch.testing.assert_close(ref, want, rtol=1e-5, atol=1e-5)
    keep = torch.ones(b, s, dtype=torch.bool)
    keep[0, 4:] = False
    masked = attention.reference(qi, ki, vi, causal=False, key_mask=keep)
    bias = keep[:, None, None, :]
    want = torch.nn.functional.scaled_dot_product_attention(qi, ki, vi, attn_mask=bias).transpose(1, 2).reshape(b, s, h * d)
    torch.testing.assert_close(masked, want, rtol=1e-5, atol=1e-5)
    assert not attention.fused_supported(qkv, d) and not attention.supported(qi, ki, vi)
    with pytest.raises(ValueError):
        attention.qkv_views(qkv, b, s, h, d, "strided")
    # the fused block ops fall back to plain arithmetic off the GPU
    x, y, z = torch.randn(4, 8), torch.randn(4, 8), torch.randn(4, 8)
    torch.testing.assert_close(nn_ops.add3(x, y, z), x + y + z)
    assert not nn_ops.parallel_norms_supported(x, torch.ones(8), torch.zeros(8), torch.ones(8), torch.zeros(8))
