"""Host-side parameter generation: Lloyd-Max codebooks and block rotations.

Same public names as the reference (src/rotorquant_vllm/quantization/__init__.py:1-5).
"""

from .isoquant import IsoQuantMSE
from .lloyd_max import LloydMaxCodebook
from .planarquant import PlanarQuantMSE

__all__ = ["LloydMaxCodebook", "IsoQuantMSE", "PlanarQuantMSE"]
