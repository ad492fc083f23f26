from .kernel import streaming_attention, streaming_attention_reference  # noqa: F401
from .varlen import streaming_attention_varlen  # noqa: F401
from .step import streaming_attention_step  # noqa: F401
from .projections import output_projection, qkv_rope_projection, rope_tables  # noqa: F401
from .fp8 import dequantize_fp8_tiles, quantize_fp8_tiles, streaming_attention_fp8  # noqa: F401
