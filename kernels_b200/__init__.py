"""kernels_b200 — B200 (sm_100a) CUDA implementation of the streaming-attention path of
``alexdremov/kernels`` behind that project's own Python operator API.

Sub-packages mirror the reference's importable packages:

* ``kernels_b200.streaming_attention`` — ``streaming_attention``, ``streaming_attention_reference``
* ``kernels_b200.self_attention`` — ``self_attention`` and its two torch references
* ``kernels_b200.softmax`` — ``softmax``

All compute goes through ``lib/libkernels_b200.so`` (C ABI in ``include/kernels_b200.h``),
built by ``python -m kernels_b200.build``.  There is no fallback when it is missing.
"""

__all__ = ["streaming_attention", "self_attention", "softmax"]
