"""Number formats and quantisation-aware training."""
from .formats import (e2m1_round, e4m3_round, e5m2_round, mxfp8_fake_quant_ref, nvfp4_fake_quant_ref, pack_fp4, unpack_fp4,  # noqa: F401
                      bf16_round, BlockScale, ScaleFactor)
from .qat import QuantSpec, cached_weight_quant, fake_quant, fake_quant_ste, new_weight_epoch  # noqa: F401
