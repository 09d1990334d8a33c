"""CPU checks of the host layer: the reference's public surface, bit accounting, constructors,
the C ABI (library loads, every declared symbol is exported, argument validation returns error
codes before anything is launched)."""
import ctypes as C
import os
import re

import pytest
import torch

import hqmq_b200 as hqmq
from hqmq_b200 import _lib, packed, quantizers

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_version_and_public_names():
    assert hqmq.__version__ == "0.1.0"
    for name in ["HQMQ", "PaddedHQMQ", "OutlierAwareHQMQQuantizer", "OutlierAwareGenericQuantizer",
                 "fused_attention", "fused_attention_reference", "with_outlier_extraction", "device_info",
                 "kernels_ada", "kernels_hopper", "kernels_blackwell"]:
        assert hasattr(hqmq, name), name
    from hqmq_b200 import kernels
    for name in ["fused_attention_ada", "fused_attention_hopper", "fused_attention_blackwell",
                 "fused_attention_reference", "decode_dequant", "encode_joint_fp8", "hopper_available",
                 "blackwell_available"]:
        assert hasattr(kernels, name), name


def test_hurwitz_units_match_oracle_order():
    from oracle import hqmq_oracle as orc
    assert torch.equal(quantizers.hurwitz_units(), orc.make_24cell())
    a = torch.randn(50, 4)
    b = torch.randn(50, 4)
    assert torch.equal(quantizers.quat_mul(a, b), orc.quat_mul(a, b))


@pytest.mark.parametrize("S,b_r,expected", [(24, 3, 3.04), (96, 4, 3.79), (192, 6, 4.54)])
def test_bits_per_value(S, b_r, expected):
    q = hqmq.HQMQ(n_layers=1, n_heads=1, secondary_size=S, radius_bits=b_r, device="cpu")
    assert abs(q.bits_per_value() - expected) < 0.01


def test_constructors_and_wrappers():
    q = hqmq.HQMQ(n_layers=4, n_heads=2, secondary_size=24, radius_bits=3, device="cpu", init="random")
    assert (q.chunk_dim, q.secondary_size, q.radius_bits) == (4, 24, 3)
    assert q.secondary_raw.shape == (4, 2, 2, 24, 4)
    w = hqmq.with_outlier_extraction(q, C=3.0)
    assert w.median_mult == 3.0 and w.threshold_mode == "median_mult" and w.inner is q
    assert w.name == "OutlierMed3_HQMQ_s24_r3"
    assert abs(w.bits_per_value() - ((1 - 0.03) * q.bits_per_value() + 0.03 * 16 + 0.25)) < 1e-9
    p = hqmq.PaddedHQMQ(n_layers=2, n_heads=2, d_head=45, secondary_size=24, radius_bits=3, device="cpu")
    assert (p.d_head_orig, p.d_head_padded, p.pad_count) == (45, 48, 3)
    with pytest.raises(ValueError):
        hqmq.HQMQ(1, 1, magnitude_mode="bogus", device="cpu")
    with pytest.raises(AssertionError):
        hqmq.OutlierAwareHQMQQuantizer(object())


def test_seeded_codebook_matches_oracle():
    from oracle import hqmq_oracle as orc
    q = hqmq.HQMQ(n_layers=2, n_heads=3, secondary_size=96, radius_bits=4, device="cpu", seed=42)
    raw = orc.secondary_raw(2, 3, 96, 42)
    assert torch.equal(q.secondary_raw.detach(), raw)
    qs, joint = q._codebook_fp32(1, 0)
    assert torch.equal(joint, orc.joint_codebook(raw[1, :, 0]))
    assert torch.equal(qs, orc.unit_secondary(raw[1, :, 0]))


def test_device_info_without_gpu():
    info = hqmq.device_info()
    assert "variant_auto_dispatched" in info and "variant" in info
    if not torch.cuda.is_available():
        assert info["variant_auto_dispatched"] == "cpu"


def test_cpu_tensors_are_rejected_loudly():
    q = hqmq.HQMQ(n_layers=1, n_heads=2, device="cpu")
    with pytest.raises(_lib.HqmqError):
        q.quantize_K(torch.randn(1, 2, 4, 16), 0)
    with pytest.raises(_lib.HqmqError):
        hqmq.fused_attention(torch.randn(1, 4, 1, 16), *[torch.zeros(1)] * 8, r_qmax=7)


def test_row_geometry():
    assert packed.idx_bits(24) == 10 and packed.idx_bits(96) == 12 and packed.idx_bits(192) == 13
    assert packed.row_bytes(32, 24, 3) == 52 and packed.row_bytes(32, 96, 4) == 64 and packed.row_bytes(32, 192, 6) == 76
    assert packed.row_bytes(16, 96, 4) == 32 and packed.row_bytes(16, 24, 3) == 28


# ---- C ABI ----------------------------------------------------------------------------------
def _declared_functions():
    hdr = open(os.path.join(ROOT, "include", "hqmq_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    return sorted(set(re.findall(r"\b(hqmq_[a-z0-9_]+)\s*\(", hdr)))


def test_library_exports_every_declared_symbol(built_lib):
    L = C.CDLL(built_lib)
    names = _declared_functions()
    assert len(names) >= 14
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/hqmq_b200.h but not exported"


def test_abi_host_helpers(built_lib):
    L = _lib.lib()
    assert L.hqmq_abi_version() == _lib.ABI_VERSION == 4
    assert L.hqmq_strerror(0) == b"ok" and b"workspace" in L.hqmq_strerror(-5)
    for n, S, b in [(32, 24, 3), (32, 96, 4), (32, 192, 6), (16, 96, 4), (12, 24, 3), (4, 24, 3)]:
        assert L.hqmq_row_bytes(n, S, b) == packed.row_bytes(n, S, b)
        assert L.hqmq_idx_bits(S) == packed.idx_bits(S)
    assert L.hqmq_row_bytes(33, 24, 3) == -2 and L.hqmq_idx_bits(4000) == -2


def test_native_index_maps_factor_the_group(built_lib):
    """ref_to_native[p] = (a << 3) | u must satisfy primary[p] = primary[u] * omega^a."""
    r2n, n2r = _lib.index_maps()
    prim = quantizers.hurwitz_units()
    omega = prim[8:9]
    powers = [prim[0:1], omega, quantizers.quat_mul(omega, omega)]
    assert sorted(r2n) == list(range(24)) and sorted(n2r) == list(range(24))
    for p in range(24):
        a, u = r2n[p] >> 3, r2n[p] & 7
        assert u < 8 and a < 3
        assert torch.allclose(quantizers.quat_mul(prim[u:u + 1], powers[a]), prim[p:p + 1], atol=1e-6)
        assert n2r[r2n[p]] == p


def test_validation_returns_error_codes_without_launching(built_lib):
    L = _lib.lib()
    assert L.hqmq_encode(None, None, 0, None) == -1
    a = _lib.EncodeArgs()
    assert L.hqmq_encode(C.byref(a), None, 0, None) == -1          # struct_size not set
    assert L.hqmq_encode_workspace_bytes(C.byref(a)) == 0
    assert L.hqmq_attn_decode(None, None, 0, None) == -1
    at = _lib.AttnArgs()
    at.struct_size = C.sizeof(_lib.AttnArgs)
    assert L.hqmq_attn_decode(C.byref(at), None, 0, None) == -1    # Q missing
    assert L.hqmq_dequant(None, None) == -1
    assert L.hqmq_combine_partials(None, 1, 1, 4, 0, 0, None, None) == -1
    assert L.hqmq_codebook_tables(None, 1, 24, None, None) == -1
    p = _lib.Packed()
    assert L.hqmq_unpack(C.byref(p), 0, 1, None, None, None, None, None) == -1


def test_packed_cache_has_no_cpu_path(built_lib):
    """The cache mirrors the reference cache's update() call but never falls back: CPU tensors raise."""
    import hqmq_b200 as hqmq
    from hqmq_b200.cache import PackedKVCache
    q = hqmq.with_outlier_extraction(hqmq.HQMQ(1, 2, 24, 3, device="cpu"), 3.0)
    cache = PackedKVCache(q, max_tokens=64, sliding_window={1: 16})
    with pytest.raises(_lib.HqmqError):
        cache.update(torch.randn(1, 2, 4, 16), torch.randn(1, 2, 4, 16), 0)
    with pytest.raises(ValueError):
        cache.update(torch.randn(1, 2, 4, 16), torch.randn(1, 2, 5, 16), 0)
    assert cache.get_seq_length(0) == 0 and cache.get_seq_length(3) == 0 and cache.compressed_bytes() >= 0
