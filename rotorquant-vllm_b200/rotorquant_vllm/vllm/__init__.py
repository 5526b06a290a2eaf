"""vLLM plugin integration of the RotorQuant attention backend.

Exports (same names as the reference, vllm/__init__.py:21-31): ``RQAttentionBackend``,
``RQFullAttentionSpec``, ``register_rq_backend``.  They are resolved on first access so that
``rotorquant_vllm.vllm.rotation`` (host-side matrix builders) can be used without importing vLLM.

The backend registers itself through the ``vllm.general_plugins`` entry point
``rotorquant_vllm.vllm:register_rq_backend``; start vLLM with ``--attention-backend CUSTOM``.
"""

__all__ = ["RQAttentionBackend", "RQFullAttentionSpec", "register_rq_backend"]


def __getattr__(name):
    if name in __all__:
        from rotorquant_vllm.vllm import rq_backend

        return getattr(rq_backend, name)
    raise AttributeError(f"module 'rotorquant_vllm.vllm' has no attribute {name!r}")
