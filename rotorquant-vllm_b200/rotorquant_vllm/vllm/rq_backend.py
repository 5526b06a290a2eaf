"""RotorQuant compressed-KV attention backend for vLLM, B200 build.

Drop-in for the reference module of the same name (src/rotorquant_vllm/vllm/rq_backend.py): the
class names, the ``CUSTOM`` registration, the environment variables and the packed uint8 cache
layout are unchanged, so vLLM sees the same plugin.  What changed is underneath: every
``forward`` runs the sm_100a kernels of librq_b200.so --

* compress-on-write   one launch writes whole cache slots (replaces two compress launches, six
                      slice assignments and a scatter, rq_backend.py:585-657 upstream);
* decode              fused paged decode for every uniform single-token batch, with the Q and
                      output rotations folded in (upstream: batch 1 only, :904, :920-935);
* prefill             fused INT8 prefill, one or several sequences (upstream: one, :957-976).

There is no Triton dispatch, no decompress-then-flash-attention path and no CPU fallback; if the
CUDA library is missing, constructing the layer fails.

Slot layout of one token (H = KV heads on this GPU, head size 128)::

    [K indices H*64 | K norms H*4 | V indices H*64 | V norms H*4 | zeros up to H*256]
"""

from __future__ import annotations

import logging
import os
from dataclasses import dataclass
from dataclasses import fields as dc_fields
from typing import TYPE_CHECKING

import torch
from vllm.v1.attention.backend import AttentionCGSupport, AttentionImplBase
from vllm.v1.attention.backends.flash_attn import (
    FlashAttentionBackend,
    FlashAttentionImpl,
    FlashAttentionMetadataBuilder,
)
from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend
from vllm.v1.kv_cache_interface import FullAttentionSpec

from rotorquant_vllm.quantization.isoquant import IsoQuantMSE
from rotorquant_vllm.quantization.planarquant import PlanarQuantMSE
from rotorquant_vllm.vllm.rotation import build_iso_R as _build_iso_R  # noqa: F401  (public name)
from rotorquant_vllm.vllm.rotation import build_planar_R as _build_planar_R  # noqa: F401
from rotorquant_vllm.vllm.rotation import build_rotation_matrix as _build_rotation_matrix

if TYPE_CHECKING:
    from vllm.v1.attention.backend import AttentionMetadataBuilder

logger = logging.getLogger(__name__)

RQ_DEFAULT_BITS = 3
RQ_DEFAULT_MODE = "iso"
RQ_SEED = 42
RQ_NORM_BYTES = 4


# ---------------------------------------------------------------------------
# Environment (same variables, same errors as upstream rq_backend.py:62-148)
# ---------------------------------------------------------------------------

def _env_choice(name: str, default: str, allowed: tuple[str, ...]) -> str:
    value = os.environ.get(name, default).lower()
    if value not in allowed:
        options = " or ".join(f"'{a}'" for a in allowed)
        raise ValueError(f"{name} must be {options}, got '{value}'")
    return value


def _env_bits(name: str, default: int) -> int:
    raw = os.environ.get(name)
    bits = int(raw) if raw else default
    if bits not in (3, 4):
        raise ValueError(f"{name} must be 3 or 4, got '{bits}'")
    return bits


def _parse_rq_mode() -> str:
    """``RQ_MODE``: 'iso' (quaternion blocks) or 'planar' (Givens blocks)."""
    return _env_choice("RQ_MODE", RQ_DEFAULT_MODE, ("iso", "planar"))


def _parse_rq_bits() -> int:
    """``RQ_BITS``: 3 or 4 bits per coordinate."""
    return _env_bits("RQ_BITS", RQ_DEFAULT_BITS)


def _parse_kv_bits() -> tuple[int, int]:
    """``RQ_K_BITS`` / ``RQ_V_BITS`` override ``RQ_BITS`` separately for keys and values."""
    default = _parse_rq_bits()
    return _env_bits("RQ_K_BITS", default), _env_bits("RQ_V_BITS", default)


def _parse_iso_mode() -> str:
    """``RQ_ISO_MODE``: 'fast' (one quaternion per block) or 'full' (two)."""
    return _env_choice("RQ_ISO_MODE", "fast", ("fast", "full"))


def _parse_rq_fused_paged_env() -> bool:
    """``RQ_USE_FUSED_PAGED`` upstream switches the fused kernels on.  Here they are the only
    path, so the variable is still parsed (truthy: 1/true/yes) but does not gate anything."""
    return os.environ.get("RQ_USE_FUSED_PAGED", "").lower() in ("1", "true", "yes")


# ---------------------------------------------------------------------------
# Kernel entry points (module-level so that tests can swap them, as upstream :118-138)
# ---------------------------------------------------------------------------

_fused_paged_kernel_available = False
_fused_paged_rq_decode_fn = None
_fused_prefill_kernel_available = False
_fused_paged_rq_int8_prefill_fn = None
_compress_and_store_fn = None
_kernel_import_error: Exception | None = None
try:
    from rotorquant_vllm import _lib as _rq_lib
    from rotorquant_vllm.cuda import compress_and_store as _compress_and_store_fn
    from rotorquant_vllm.cuda import fused_paged_rq_decode as _fused_paged_rq_decode_fn

    _rq_lib.lib()
    _fused_paged_kernel_available = True
    logger.info("RotorQuant CUDA library loaded: %s", _rq_lib.lib().rq_version().decode())
except (ImportError, RuntimeError, OSError) as exc:  # library not built
    _kernel_import_error = exc
    logger.info("Fused paged RQ decode kernel unavailable: %s", exc)

try:
    from rotorquant_vllm.cuda.prefill import (
        fused_paged_rq_int8_prefill as _fused_paged_rq_int8_prefill_fn,
    )

    _fused_prefill_kernel_available = _fused_paged_kernel_available
except (ImportError, RuntimeError, OSError) as exc:
    logger.info("Fused paged RQ int8 prefill kernel unavailable: %s", exc)


# ---------------------------------------------------------------------------
# Cache sizing (upstream :155-188)
# ---------------------------------------------------------------------------

def _rq_bytes_per_component(head_dim: int, num_kv_heads: int) -> int:
    """Bytes of K (or V) for one token: two 4-bit indices per byte plus one fp32 norm per head."""
    return num_kv_heads * (head_dim // 2 + RQ_NORM_BYTES)


def _rq_bytes_per_token_kv(head_dim: int, num_kv_heads: int) -> int:
    """Payload bytes of one token, K and V (8 heads x 128: 1088, against 4096 in fp16)."""
    return 2 * _rq_bytes_per_component(head_dim, num_kv_heads)


def _rq_padded_slot_bytes(head_dim: int) -> int:
    """Per-head slot size: the one-head payload rounded up to a power of two, so that RQ pages
    divide evenly into the pages of other layer types in hybrid models."""
    raw = _rq_bytes_per_token_kv(head_dim, 1)
    return 1 << (raw - 1).bit_length()


def _rq_total_bytes(head_dim: int, num_kv_heads: int) -> int:
    """Allocated bytes of one token slot."""
    return num_kv_heads * _rq_padded_slot_bytes(head_dim)


@dataclass(frozen=True, kw_only=True)
class RQFullAttentionSpec(FullAttentionSpec):
    """Full-attention KV spec whose page size is the RotorQuant slot size (``dtype=torch.uint8``)."""

    @property
    def real_page_size_bytes(self) -> int:  # noqa: D102
        return self.block_size * _rq_total_bytes(self.head_size, self.num_kv_heads)


class RQMetadataBuilder(FlashAttentionMetadataBuilder):
    """FlashAttention's metadata builder with RotorQuant's CUDA-graph capability."""

    @classmethod
    def get_cudagraph_support(cls, vllm_config: object, kv_cache_spec: object) -> AttentionCGSupport:
        """Single-token decode is capturable: the compress and decode launches read no device
        metadata on the host, allocate nothing and use fixed grids."""
        if _fused_paged_kernel_available:
            return AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE
        return AttentionCGSupport.NEVER


class RQAttentionBackend(FlashAttentionBackend):
    """Attention backend with a RotorQuant-compressed paged KV cache, registered as ``CUSTOM``."""

    forward_includes_kv_cache_update = True

    @classmethod
    def supports_mm_prefix(cls) -> bool:
        return True

    @staticmethod
    def get_name() -> str:
        return "CUSTOM"

    @staticmethod
    def get_impl_cls() -> type[AttentionImplBase]:
        return RQAttentionImpl

    @staticmethod
    def get_builder_cls() -> type[AttentionMetadataBuilder]:
        return RQMetadataBuilder

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto") -> tuple[int, ...]:
        """``(num_blocks, block_size, total_bytes)`` uint8; see the module docstring for a slot."""
        return (num_blocks, block_size, _rq_total_bytes(head_size, num_kv_heads))

    @staticmethod
    def get_kv_cache_stride_order(include_num_layers_dimension: bool = False) -> tuple[int, ...]:
        """No custom stride order: raising makes vLLM keep the identity layout."""
        raise NotImplementedError


class RQAttentionImpl(FlashAttentionImpl):
    """Attention layer implementation over the compressed cache.

    ``forward`` (1) compresses the step's new K/V tokens straight into their cache slots and
    (2) attends over the compressed cache in rotated space: uniform single-token batches go to
    the fused decode kernel, everything else to the fused INT8 prefill kernel.
    """

    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        if not _fused_paged_kernel_available:
            raise RuntimeError(
                "RotorQuant CUDA library is not available and this build has no other path: "
                f"{_kernel_import_error}")

        self._rq_mode = _parse_rq_mode()
        iso_mode = _parse_iso_mode()
        self._k_bits, self._v_bits = _parse_kv_bits()

        from vllm.config import get_current_vllm_config_or_none

        vllm_config = get_current_vllm_config_or_none()
        device = vllm_config.device_config.device if vllm_config is not None else torch.device("cpu")

        def make(bits: int):
            if self._rq_mode == "iso":
                return IsoQuantMSE(self.head_size, bits, seed=RQ_SEED, mode=iso_mode, device=device)
            return PlanarQuantMSE(self.head_size, bits, seed=RQ_SEED, device=device)

        # K and V share the seed, hence the rotation, even with different bit widths.
        self._k_quantizer = make(self._k_bits)
        self._v_quantizer = self._k_quantizer if self._v_bits == self._k_bits else make(self._v_bits)

        rot = _build_rotation_matrix(self._k_quantizer, self.head_size, device)
        # Structure check with its one host copy happens here, at build time; the launchers then
        # recognise the matrix by identity and never synchronise on the request path.
        from rotorquant_vllm.cuda.rotation import validate_rotation

        validate_rotation(rot)
        self._rq_rot = rot
        self._rq_rot_T = rot.T.contiguous()
        self._rq_rot_T_even = self._rq_rot_T[:, 0::2].contiguous()
        self._rq_rot_T_odd = self._rq_rot_T[:, 1::2].contiguous()
        self._half_d = self.head_size // 2
        self._set_layout()

        self._cg_buffers_ready = False
        self._max_model_len = vllm_config.model_config.max_model_len if vllm_config is not None else 8192
        self._max_prefill_len = (vllm_config.scheduler_config.max_num_batched_tokens
                                 if vllm_config is not None else 2048)
        self._max_num_seqs = (vllm_config.scheduler_config.max_num_seqs if vllm_config is not None else 256)
        _parse_rq_fused_paged_env()
        self._fused_paged_available = _fused_paged_kernel_available
        self._fused_prefill_available = _fused_prefill_kernel_available

        fp16_bytes = 2 * self.num_kv_heads * self.head_size * 2
        logger.info(
            "RQAttentionImpl: %s mode, %d KV heads, head_size=%d, k_bits=%d, v_bits=%d, "
            "%d bytes/token (%.2fx compression vs FP16)",
            self._rq_mode, self.num_kv_heads, self.head_size, self._k_bits, self._v_bits,
            self._total_bytes, fp16_bytes / self._total_bytes)
        logger.info("Fused paged RQ decode: %s; fused paged RQ int8 prefill: %s",
                    "enabled" if self._fused_paged_available else "disabled",
                    "enabled" if self._fused_prefill_available else "disabled")

    def _set_layout(self) -> None:
        h, half = self.num_kv_heads, self.head_size // 2
        self._k_idx_end = h * half
        self._k_norm_end = self._k_idx_end + h * RQ_NORM_BYTES
        self._v_idx_end = self._k_norm_end + h * half
        self._v_norm_end = self._v_idx_end + h * RQ_NORM_BYTES
        self._total_bytes = _rq_total_bytes(self.head_size, h)

    def _init_cg_buffers(self, kv_cache: torch.Tensor, compute_dtype: torch.dtype) -> None:
        """Reserve the scratch of both kernels once, before serving starts, so that no ``forward``
        allocates later (for instance inside a CUDA graph capture): the decode scratch for the
        largest batch the scheduler admits (``max_num_seqs``) at the longest context the cache can
        hold, and the prefill staging buffer for one batch of ``max_num_batched_tokens`` tokens
        (bounded by the launcher's cap; larger batches take the kernel that needs no scratch)."""
        from rotorquant_vllm.cuda.decode import reserve_decode_workspace
        from rotorquant_vllm.cuda.prefill import reserve_prefill_scratch

        num_blocks, block_size, _ = kv_cache.shape
        max_tokens = min(self._max_model_len, num_blocks * block_size)
        # the launcher bounds sequence lengths by (block-table width x block size): whole blocks
        max_tokens = (max_tokens + block_size - 1) // block_size * block_size
        reserve_decode_workspace(kv_cache.device, max(1, self._max_num_seqs), self.num_heads, self.num_kv_heads,
                                 self.head_size, max_tokens)
        lib = _rq_lib.lib()
        prefill_seqs = max(1, min(self._max_num_seqs, self._max_prefill_len // 128 + 1))
        reserve_prefill_scratch(kv_cache.device,
                                lib.rq_prefill_workspace_bytes(prefill_seqs, self.num_kv_heads, self._max_prefill_len))
        self._cg_buffers_ready = True

    # -- cache write -------------------------------------------------------------------------

    def _compress_and_store(self, key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
                            slot_mapping: torch.Tensor, compress_out=None, row_out=None) -> None:
        """Compress ``(N, H, D)`` keys and values and write their slots (one kernel launch).

        ``compress_out`` / ``row_out`` are accepted for signature compatibility with upstream
        (:585-593); the fused kernel needs no intermediate buffers.
        """
        _compress_and_store_fn(key, value, kv_cache, slot_mapping, self._rq_rot,
                               self._k_quantizer.boundaries, self._v_quantizer.boundaries)

    # -- decompress (for callers that want plain K/V tensors; attention itself never decompresses) --

    def _decompress_cache(self, kv_cache: torch.Tensor, compute_dtype: torch.dtype):
        """The whole cache as ``(NB, BS, H, D)`` K and V in ``compute_dtype``, rotated space
        (upstream :663-735), in one launch."""
        from rotorquant_vllm.cuda.decompress import decompress_blocks

        return decompress_blocks(kv_cache, None, self.num_kv_heads, self._k_quantizer.centroids,
                                 self._v_quantizer.centroids, compute_dtype)

    def _decompress_cache_paged(self, kv_cache: torch.Tensor, block_table: torch.Tensor,
                                seq_lens: torch.Tensor, compute_dtype: torch.dtype, out_k=None, out_v=None):
        """Only the physical blocks ``block_table`` references: ``(key_cache, value_cache,
        remapped_block_table)`` as upstream (:737-852).  ``out_k`` / ``out_v`` ``(max_tokens, H, D)``
        receive the rows when they are large enough, as upstream."""
        from rotorquant_vllm.cuda.decompress import decompress_cache_paged

        k, v, remapped = decompress_cache_paged(kv_cache, block_table, seq_lens, self.num_kv_heads,
                                                self._k_quantizer.centroids, self._v_quantizer.centroids,
                                                compute_dtype)
        tokens = k.shape[0] * k.shape[1]
        if out_k is not None and out_k.shape[0] >= tokens:
            out_k[:tokens].copy_(k.reshape(tokens, *k.shape[2:]))
            k = out_k[:tokens].reshape(k.shape)
        if out_v is not None and out_v.shape[0] >= tokens:
            out_v[:tokens].copy_(v.reshape(tokens, *v.shape[2:]))
            v = out_v[:tokens].reshape(v.shape)
        return k, v, remapped

    # -- forward -------------------------------------------------------------------------------

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None,
                output_scale=None, output_block_scale=None):
        """Write the new tokens into the compressed cache, then attend over it.

        ``query (T, H_Q, D)``, ``key``/``value (T, H, D)`` or None, ``kv_cache`` uint8
        ``(num_blocks, block_size, total_bytes)``; the result is written into ``output``.
        """
        assert output is not None, "Output tensor must be provided."
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError(
                "Fused output quantization is not supported with RotorQuant backend")
        if attn_metadata is None or kv_cache is None:
            return output.zero_()

        from vllm.v1.attention.backend import AttentionType

        n = attn_metadata.num_actual_tokens
        if self.attn_type in (AttentionType.ENCODER_ONLY, AttentionType.ENCODER):
            return self._forward_encoder_attention(query[:n], key[:n], value[:n], output[:n],
                                                   attn_metadata, layer)

        if not self._cg_buffers_ready:
            self._init_cg_buffers(kv_cache, query.dtype)
        if key is not None and value is not None:
            self._compress_and_store(key, value, kv_cache, attn_metadata.slot_mapping)

        seq_lens = attn_metadata.seq_lens
        num_seqs = seq_lens.numel()
        # One query token per sequence: upstream only recognises a single-token batch (:904);
        # any batch whose longest query is one token takes the same kernel here.
        is_decode = n == 1 or (n == num_seqs and getattr(attn_metadata, "max_query_len", None) == 1)
        common = (kv_cache, attn_metadata.block_table, seq_lens, self._k_quantizer.centroids,
                  self._v_quantizer.centroids, self._rq_rot, self.num_kv_heads, self.head_size,
                  kv_cache.shape[1])

        if is_decode:
            if not self._fused_paged_available:
                raise RuntimeError("RotorQuant fused decode kernel is not available")
            _fused_paged_rq_decode_fn(query[:n], *common, sm_scale=self.scale, out=output[:n])
            return output

        if getattr(attn_metadata, "use_cascade", False):
            raise NotImplementedError("RQ does not yet support cascade attention")
        if not self._fused_prefill_available:
            raise RuntimeError("RotorQuant fused prefill kernel is not available")
        extra = {}
        if num_seqs != 1:
            extra["cu_seqlens_q"] = attn_metadata.query_start_loc
        # host-side bounds from the metadata: they size the grid and the scratch of the staged path
        if getattr(attn_metadata, "max_query_len", None):
            extra["max_q_len"] = int(attn_metadata.max_query_len)
        if getattr(attn_metadata, "max_seq_len", None):
            extra["max_seq_len"] = int(attn_metadata.max_seq_len)
        _fused_paged_rq_int8_prefill_fn(query[:n], *common, sm_scale=self.scale, out=output[:n],
                                        **extra)
        return output


# ---------------------------------------------------------------------------
# Registration (upstream :1046-1093)
# ---------------------------------------------------------------------------

_original_get_kv_cache_spec = None


def register_rq_backend() -> None:
    """Register the backend as ``AttentionBackendEnum.CUSTOM`` and make decoder attention layers
    report :class:`RQFullAttentionSpec` (uint8 pages of RotorQuant size).

    Runs automatically through the ``vllm.general_plugins`` entry point; call it by hand before
    starting vLLM with ``--attention-backend CUSTOM`` otherwise.
    """
    global _original_get_kv_cache_spec  # noqa: PLW0603

    register_backend(AttentionBackendEnum.CUSTOM,
                     "rotorquant_vllm.vllm.rq_backend.RQAttentionBackend")

    # The KV-cache manager table is keyed by exact spec type.
    from vllm.v1.core.single_type_kv_cache_manager import spec_manager_map

    spec_manager_map.setdefault(RQFullAttentionSpec, spec_manager_map[FullAttentionSpec])

    from vllm.model_executor.layers.attention.attention import Attention

    if _original_get_kv_cache_spec is None:
        _original_get_kv_cache_spec = Attention.get_kv_cache_spec

    def _rq_get_kv_cache_spec(self, vllm_config):
        spec = _original_get_kv_cache_spec(self, vllm_config)
        if type(spec) is not RQFullAttentionSpec and isinstance(spec, FullAttentionSpec):
            values = {f.name: getattr(spec, f.name) for f in dc_fields(spec)}
            values["dtype"] = torch.uint8
            return RQFullAttentionSpec(**values)
        return spec

    Attention.get_kv_cache_spec = _rq_get_kv_cache_spec
    logger.info("RQ attention backend registered as CUSTOM (compressed cache)")
