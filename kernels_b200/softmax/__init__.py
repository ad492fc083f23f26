from .kernel import softmax, softmax_naive  # noqa: F401
