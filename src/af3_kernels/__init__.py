"""Import-name compatibility: ``import af3_kernels`` (with ``src/`` on the path, as in the
reference's layout) resolves to the B200 package.  Everything lives in ``af3_kernels_b200``."""
import os as _os
import sys as _sys

_root = _os.path.dirname(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))
if _root not in _sys.path:
    _sys.path.insert(0, _root)

from af3_kernels_b200 import *  # noqa: F401,F403
from af3_kernels_b200 import (  # noqa: F401
    _attention_cpp,
    dot_product_attention_cpp,
    gated_linear_unit_cpp,
    pad_and_align_tensor,
    print_debug_thread_imbalance,
    print_debug_timers,
    reset_debug_timers,
    self_attention_cpp,
    vnni_repack_tensor,
)
