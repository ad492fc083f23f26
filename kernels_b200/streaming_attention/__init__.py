from .kernel import streaming_attention, streaming_attention_reference  # noqa: F401
from .varlen import streaming_attention_varlen  # noqa: F401
from .step import streaming_attention_step  # noqa: F401
