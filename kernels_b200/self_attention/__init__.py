from .kernel import self_attention  # noqa: F401
from .kernel import self_attention_reference, self_attention_reference_naive  # noqa: F401
