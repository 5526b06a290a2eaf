"""RotorQuant KV-cache compression for vLLM -- B200-native hot path.

Same import name and public names as the reference package
(src/rotorquant_vllm/__init__.py:20-30), so the vLLM entry point
``rotorquant_vllm.vllm:register_rq_backend`` keeps working.  The vLLM-facing
names are resolved lazily: importing the kernel launchers
(``rotorquant_vllm.cuda``) or the host-side parameter generators
(``rotorquant_vllm.quantization``) does not import vLLM.
"""

__all__ = [
    "IsoQuantMSE",
    "LloydMaxCodebook",
    "PlanarQuantMSE",
    "RQAttentionBackend",
    "RQFullAttentionSpec",
    "register_rq_backend",
]

_QUANT = {"IsoQuantMSE", "LloydMaxCodebook", "PlanarQuantMSE"}
_VLLM = {"RQAttentionBackend", "RQFullAttentionSpec", "register_rq_backend"}


def __getattr__(name):
    if name in _QUANT:
        from rotorquant_vllm import quantization

        return getattr(quantization, name)
    if name in _VLLM:
        from rotorquant_vllm import vllm as _v

        return getattr(_v, name)
    raise AttributeError(f"module 'rotorquant_vllm' has no attribute {name!r}")
