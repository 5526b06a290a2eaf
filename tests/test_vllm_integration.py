"""The vLLM-facing plugin surface: registration, cache layout, environment variables and the
way ``forward`` dispatches to the kernel entry points.  Runs without a GPU (the kernels are
replaced by recording stand-ins, the technique the reference's own tests use,
tests/test_vllm_integration.py:109-239).
"""

from types import SimpleNamespace

import pytest
import torch

vllm = pytest.importorskip("vllm")

import rotorquant_vllm.vllm.rq_backend as backend  # noqa: E402
from rotorquant_vllm.quantization import IsoQuantMSE, PlanarQuantMSE  # noqa: E402
from rotorquant_vllm.vllm import (  # noqa: E402
    RQAttentionBackend,
    RQFullAttentionSpec,
    register_rq_backend,
)
from vllm.v1.attention.backend import AttentionType  # noqa: E402
from vllm.v1.attention.backends.registry import AttentionBackendEnum  # noqa: E402


# ---- registration -------------------------------------------------------------------------

def test_registration_overrides_custom_backend():
    register_rq_backend()
    assert AttentionBackendEnum.CUSTOM.is_overridden()
    assert "rotorquant_vllm" in AttentionBackendEnum.CUSTOM.get_path()
    register_rq_backend()  # idempotent


def test_backend_identity():
    assert RQAttentionBackend.get_name() == "CUSTOM"
    assert RQAttentionBackend.get_impl_cls() is backend.RQAttentionImpl
    assert RQAttentionBackend.get_builder_cls() is backend.RQMetadataBuilder
    assert RQAttentionBackend.supports_mm_prefix() is True
    assert RQAttentionBackend.forward_includes_kv_cache_update is True
    with pytest.raises(NotImplementedError):
        RQAttentionBackend.get_kv_cache_stride_order()


# ---- layout ---------------------------------------------------------------------------------

@pytest.mark.parametrize("heads,raw,total", [(8, 1088, 2048), (4, 544, 1024), (1, 136, 256)])
def test_slot_sizes(heads, raw, total):
    assert backend._rq_bytes_per_token_kv(128, heads) == raw
    assert backend._rq_padded_slot_bytes(128) == 256
    assert backend._rq_total_bytes(128, heads) == total


def test_cache_shape_and_page_size():
    assert RQAttentionBackend.get_kv_cache_shape(100, 16, 8, 128) == (100, 16, 2048)
    spec = RQFullAttentionSpec(block_size=16, num_kv_heads=8, head_size=128, dtype=torch.uint8)
    assert spec.real_page_size_bytes == 32768


def test_compression_ratio_bounds():
    ratio = (2 * 8 * 128 * 2) / backend._rq_bytes_per_token_kv(128, 8)
    assert 3.5 < ratio < 4.0


# ---- environment ------------------------------------------------------------------------------

def test_environment_defaults(monkeypatch):
    for v in ("RQ_MODE", "RQ_BITS", "RQ_K_BITS", "RQ_V_BITS", "RQ_ISO_MODE", "RQ_USE_FUSED_PAGED"):
        monkeypatch.delenv(v, raising=False)
    assert backend._parse_rq_mode() == "iso"
    assert backend._parse_rq_bits() == 3
    assert backend._parse_kv_bits() == (3, 3)
    assert backend._parse_iso_mode() == "fast"
    assert backend._parse_rq_fused_paged_env() is False


def test_environment_overrides_and_errors(monkeypatch):
    monkeypatch.setenv("RQ_MODE", "PLANAR")
    monkeypatch.setenv("RQ_BITS", "4")
    monkeypatch.setenv("RQ_V_BITS", "3")
    monkeypatch.setenv("RQ_ISO_MODE", "full")
    monkeypatch.setenv("RQ_USE_FUSED_PAGED", "Yes")
    assert backend._parse_rq_mode() == "planar"
    assert backend._parse_kv_bits() == (4, 3)
    assert backend._parse_iso_mode() == "full"
    assert backend._parse_rq_fused_paged_env() is True
    for var, bad in (("RQ_MODE", "rotor"), ("RQ_BITS", "5"), ("RQ_K_BITS", "2"), ("RQ_ISO_MODE", "slow")):
        monkeypatch.setenv(var, bad)
        with pytest.raises(ValueError, match=var):
            {"RQ_MODE": backend._parse_rq_mode, "RQ_BITS": backend._parse_rq_bits,
             "RQ_K_BITS": backend._parse_kv_bits, "RQ_ISO_MODE": backend._parse_iso_mode}[var]()
        monkeypatch.delenv(var)


# ---- rotation matrices --------------------------------------------------------------------------

@pytest.mark.parametrize("make", [
    lambda: (IsoQuantMSE(128, 3, seed=42, mode="fast"), "fast"),
    lambda: (IsoQuantMSE(128, 3, seed=42, mode="full"), "full"),
])
def test_iso_rotation_is_orthogonal(make):
    q, mode = make()
    R = backend._build_iso_R(q, 128, "cpu", mode)
    assert (R @ R.T - torch.eye(128)).abs().max().item() < 1e-5
    assert torch.equal(R, backend._build_rotation_matrix(q, 128, "cpu"))


def test_planar_rotation_is_orthogonal():
    R = backend._build_planar_R(PlanarQuantMSE(128, 3, seed=42), 128, "cpu")
    assert (R @ R.T - torch.eye(128)).abs().max().item() < 1e-5


# ---- forward dispatch -------------------------------------------------------------------------------

def _bare_impl():
    impl = backend.RQAttentionImpl.__new__(backend.RQAttentionImpl)
    impl.attn_type = AttentionType.DECODER
    impl._cg_buffers_ready = True
    impl._fused_paged_available = True
    impl._fused_prefill_available = True
    impl.num_kv_heads = 8
    impl.head_size = 128
    impl.block_size = 16
    impl.scale = 0.125
    impl._k_quantizer = SimpleNamespace(centroids=torch.randn(8), boundaries=torch.randn(7))
    impl._v_quantizer = SimpleNamespace(centroids=torch.randn(16), boundaries=torch.randn(15))
    impl._rq_rot = torch.eye(128)
    return impl


def _recorder(log, fill):
    def fn(q, kv_cache, block_table, seq_lens, centroids_k, centroids_v, rotation, num_kv_heads,
           head_dim, block_size, sm_scale=None, out=None, **extra):
        log.append(dict(q=tuple(q.shape), kv=tuple(kv_cache.shape), bt=tuple(block_table.shape),
                        seq_lens=seq_lens.clone(), nk=centroids_k.numel(), nv=centroids_v.numel(),
                        heads=num_kv_heads, dim=head_dim, bs=block_size, scale=sm_scale,
                        extra=sorted(extra)))
        out.fill_(fill)
        return out
    return fn


def test_single_token_decode_goes_to_the_decode_kernel(monkeypatch):
    log = []
    monkeypatch.setattr(backend, "_fused_paged_rq_decode_fn", _recorder(log, 3.0))
    impl = _bare_impl()
    query = torch.randn(1, 8, 128, dtype=torch.bfloat16)
    out = torch.zeros_like(query)
    md = SimpleNamespace(num_actual_tokens=1, block_table=torch.zeros(1, 4, dtype=torch.int32),
                         seq_lens=torch.tensor([1], dtype=torch.int32))
    res = impl.forward(None, query, None, None, torch.zeros(4, 16, 2048, dtype=torch.uint8), md,
                       output=out)
    assert res is out and torch.all(out == 3.0)
    (call,) = log
    assert call["q"] == (1, 8, 128) and call["kv"] == (4, 16, 2048) and call["bt"] == (1, 4)
    assert (call["heads"], call["dim"], call["bs"], call["scale"]) == (8, 128, 16, 0.125)
    assert (call["nk"], call["nv"]) == (8, 16)


def test_batched_decode_goes_to_the_decode_kernel_and_writes_the_cache_first(monkeypatch):
    log, stores = [], []
    monkeypatch.setattr(backend, "_fused_paged_rq_decode_fn", _recorder(log, 2.0))
    monkeypatch.setattr(backend, "_compress_and_store_fn",
                        lambda k, v, cache, slots, rot, kb, vb: stores.append(
                            (tuple(k.shape), slots.tolist(), kb.numel(), vb.numel(), len(log))))
    impl = _bare_impl()
    query = torch.randn(6, 8, 128, dtype=torch.bfloat16)   # padded to 6, 5 real tokens
    kv = torch.randn(6, 8, 128, dtype=torch.bfloat16)
    out = torch.zeros_like(query)
    md = SimpleNamespace(num_actual_tokens=5, max_query_len=1, slot_mapping=torch.arange(5),
                         block_table=torch.zeros(5, 4, dtype=torch.int32),
                         seq_lens=torch.full((5,), 9, dtype=torch.int32))
    impl.forward(None, query, kv, kv, torch.zeros(4, 16, 2048, dtype=torch.uint8), md, output=out)
    assert stores == [((6, 8, 128), [0, 1, 2, 3, 4], 7, 15, 0)]      # stored before attention
    assert log[0]["q"] == (5, 8, 128)
    assert torch.all(out[:5] == 2.0) and torch.all(out[5] == 0)


def test_single_sequence_prefill_goes_to_the_int8_kernel(monkeypatch):
    log = []
    monkeypatch.setattr(backend, "_fused_paged_rq_int8_prefill_fn", _recorder(log, 5.0))
    impl = _bare_impl()
    impl._fused_paged_available = False
    query = torch.randn(3, 8, 128, dtype=torch.bfloat16)
    out = torch.zeros_like(query)
    md = SimpleNamespace(num_actual_tokens=3, block_table=torch.zeros(1, 4, dtype=torch.int32),
                         seq_lens=torch.tensor([3], dtype=torch.int32), use_cascade=False,
                         slot_mapping=torch.arange(3))
    res = impl.forward(None, query, None, None, torch.zeros(4, 16, 2048, dtype=torch.uint8), md,
                       output=out)
    assert res is out and torch.all(out == 5.0)
    assert log[0]["q"] == (3, 8, 128) and log[0]["extra"] == []
    assert torch.equal(log[0]["seq_lens"], torch.tensor([3], dtype=torch.int32))


def test_multi_sequence_prefill_passes_query_start_loc(monkeypatch):
    log = []
    monkeypatch.setattr(backend, "_fused_paged_rq_int8_prefill_fn", _recorder(log, 1.0))
    impl = _bare_impl()
    query = torch.randn(7, 8, 128, dtype=torch.bfloat16)
    md = SimpleNamespace(num_actual_tokens=7, max_query_len=4, use_cascade=False,
                         query_start_loc=torch.tensor([0, 4, 7], dtype=torch.int32),
                         block_table=torch.zeros(2, 4, dtype=torch.int32),
                         seq_lens=torch.tensor([4, 20], dtype=torch.int32))
    impl.forward(None, query, None, None, torch.zeros(4, 16, 2048, dtype=torch.uint8), md,
                 output=torch.zeros_like(query))
    assert log[0]["extra"] == ["cu_seqlens_q", "max_q_len"]
    md.max_seq_len = 20
    impl.forward(None, query, None, None, torch.zeros(4, 16, 2048, dtype=torch.uint8), md,
                 output=torch.zeros_like(query))
    assert log[1]["extra"] == ["cu_seqlens_q", "max_q_len", "max_seq_len"]


def test_forward_edge_cases(monkeypatch):
    impl = _bare_impl()
    query = torch.randn(2, 8, 128, dtype=torch.bfloat16)
    out = torch.ones_like(query)
    assert torch.all(impl.forward(None, query, None, None, None, None, output=out) == 0)
    with pytest.raises(NotImplementedError):
        impl.forward(None, query, None, None, None, None, output=out, output_scale=torch.ones(1))
    with pytest.raises(AssertionError):
        impl.forward(None, query, None, None, None, None)
    md = SimpleNamespace(num_actual_tokens=2, use_cascade=True, max_query_len=2,
                         block_table=torch.zeros(1, 4, dtype=torch.int32),
                         seq_lens=torch.tensor([2], dtype=torch.int32))
    with pytest.raises(NotImplementedError, match="cascade"):
        impl.forward(None, query, None, None, torch.zeros(4, 16, 2048, dtype=torch.uint8), md,
                     output=out)
