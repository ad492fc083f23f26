from .kernel import streaming_attention, streaming_attention_reference  # noqa: F401
