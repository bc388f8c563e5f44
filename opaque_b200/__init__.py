"""opaque_b200 — a B200-native differentially-private training framework.

Public namespaces mirror the reference's ``opaque.*`` layout (``serialization``,
``types``, ``pytree``, ``random``, ``functional``, ``distributed``, ``profiling``,
``precision``, ``scheduling``, ``device``, ``accounting``, ``dpsgd``, ``dpftrl``,
``optimizers``, ``patches``, ``transformers``, ``alignment``, ``auditing``) and add
the B200 layers: ``ops`` (hand-written sm_100a kernels), ``parallel``
(peer-memory reduce-scatter / all-gather and the sharded noise+optimizer step),
``engine`` (reference and fused DP gradient engines) and ``models``.
"""
__version__ = "0.2.0"

from .serialization import _tensors as _tensor_serializers  # noqa: E402,F401  (registers tensor / array leaves)
