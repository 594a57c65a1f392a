"""PyTorch specification of the K2 pack step under the module name the reference uses
(``terrace/ops/k2_ref.py``); the implementation lives in ``ops/refs.py``."""
from .refs import fixed_hist, k2_pack_ref, stable_bucket_order  # noqa: F401
