"""tpa_b200 — Tensor Product Attention forward and ring forward on B200 (sm_100a).

Drop-in for the forward path of jondeaton/tensor-product-attention-jax over
hand-written CUDA behind a C ABI (include/tpa_b200.h).  The module layout follows the
reference: `tpa_b200.tpa.tpa(...)` for tpa/tpa.py and
`tpa_b200.ring_tpa.ring_tpa(...)` / `ring_tp_self_attention(...)` for tpa/ring_tpa.py.
Importing this package loads libtpa_b200.so and raises if it has not been built: there
is no CPU or PyTorch fallback.
"""

from . import _capi  # noqa: F401  (loads the shared library or raises)
from . import tpa, ring_tpa, mha  # noqa: F401

__all__ = ["tpa", "ring_tpa", "mha"]
