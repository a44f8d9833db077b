"""KV page metadata, precision tiers, quantisers (KIVI / FWHT / RaBitQ-style residual), TurboQuant runtime,
dual-track pool and the optimisation decision matrix."""
from .header import (KV_PAGE_HEADER_DTYPE, CompressionCodec, KvPageHeaderTable, KvPageLayout, PrecisionTier,  # noqa: F401
                     StorageTier, DoubleBufferedKvState)
from .quant import (fwht, kivi_dequantize, kivi_quantize_k, kivi_quantize_v, fp8_quantize_page, fp8_dequantize_page,  # noqa: F401
                    stochastic_round, KiviPage)
from .turboquant import TurboQuantConfig, TurboQuantRuntime  # noqa: F401
from .dual_track import DualTrackPool  # noqa: F401
from .decision import KvDecisionMatrix, KvVariant, HardwareProfile  # noqa: F401
